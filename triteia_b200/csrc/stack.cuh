// Per-row fp32 checksum of an fp16 matrix: sums[r] (+)= sum over n of y[r, n].
// The linear-stack scenario (many independent indexed delta matmuls over the same routed tokens)
// reduces every linear's output to one number per token, so that the result a token owner gets back
// covers all of them without shipping every output row.  One warp per row, 16-byte loads, fp32 adds
// in a fixed order (lane-strided partial sums, then a butterfly), so results are run-to-run identical.
// The reference has no counterpart (its benchmarks compare full outputs, one linear at a time).
#pragma once

#include "common.cuh"

namespace trb {

__global__ void row_checksum_kernel(const uint4* __restrict__ y, float* __restrict__ sums, int rows, int n_vec,
                                    int accumulate, const int* __restrict__ row_map,
                                    const int* __restrict__ first_row) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  if (first_row != nullptr && warp < *first_row) return;   // sorted order: rows without a delta come first and hold nothing
  const uint4* row = y + (size_t)warp * n_vec;
  float acc = 0.f;
  for (int i = lane; i < n_vec; i += 32) {
    const uint4 v = row[i];
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __half22float2(h[e]);
      acc += f.x;
      acc += f.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    const int out = row_map ? row_map[warp] : warp;      // row r of y is row row_map[r] of the caller's order
    if (out >= 0 && out < rows) sums[out] = accumulate ? sums[out] + acc : acc;
  }
}

}  // namespace trb

namespace trb {
static int row_checksum_launch(const void* y, void* sums, int rows, int prob_m, int accumulate, const int* row_map,
                               const int* first_row, cudaStream_t stream) {
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3((rows + 7) / 8);
  lc.blockDim = dim3(256);
  lc.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits before it reads y
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return cudaLaunchKernelEx(&lc, row_checksum_kernel, (const uint4*)y, (float*)sums, rows, prob_m / 8, accumulate,
                            row_map, first_row) == cudaSuccess
             ? TRB_OK
             : TRB_ERR_CUDA;
}
}  // namespace trb

extern "C" int trb_row_checksum(const void* y, void* sums, int rows, int prob_m, int accumulate, int dev,
                                void* stream) {
  using namespace trb;
  if (rows <= 0) return TRB_OK;
  if (!y || !sums) return TRB_ERR_BAD_ARG;
  if (prob_m <= 0 || prob_m % 8 != 0 || (reinterpret_cast<uintptr_t>(y) & 15) != 0) return TRB_ERR_PROB_SHAPE;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  return row_checksum_launch(y, sums, rows, prob_m, accumulate, nullptr, nullptr, (cudaStream_t)stream);
}

// Working memory of trb_stack_pass for `rows` rows over `num_deltas` deltas: router counters, the
// permutation, the two tile lists and the partial tiles of the tail K split.
extern "C" size_t trb_stack_scratch_bytes(int rows, int num_deltas) {
  if (rows <= 0 || num_deltas <= 0) return kCounterBytes;
  return kCounterBytes + align_up((size_t)rows * 4, 256) + 3 * align_up(small_tile_capacity(rows, num_deltas) * 4, 256) +
         3 * align_up(big_tile_capacity(rows) * 4, 256) + kKsplitBufBytes;
}

// One pass of a stack of independent delta linears over one routed batch, issued from C with no host
// read in between (a Python call per launch costs more than most of these kernels run, and a host
// read of segment counts leaves the GPU idle).  ids[r] in [0, num_deltas) selects the delta of row r
// in EVERY linear (any other id: the row has no delta, its outputs count as zero), so the rows are routed once: one router launch (permutation + the two tile lists of
// trb_sbmm_indexed), one row gather per input width, then per linear the tcgen05 launch (long
// segments; only for batches of more than 128 rows), the mma.sp launch (8-token tiles, tail K split)
// and the fold of the linear's output into the per-row fp32 checksum.  Arrays are host arrays; the
// pointers in them are device pointers.
//   x_of_width[w]    [rows, width[w]] fp16, caller's row order;  xs_of_width[w] same size, scratch
//   k[i], n[i]       shape of linear i; k[i] must be one of width[]
//   y_of[i]          [rows, n[i]] fp16 scratch (sorted row order; buffers may be shared between
//                    linears of one n: the checksum is taken before the next linear overwrites it)
//   y_last           [rows, n[n_linears - 1]] fp16, output of the last linear in the caller's row order
//   checksum         [rows] fp32 in the caller's row order; the pass ADDS to it (zero it first)
// No counterpart in the reference.
extern "C" int trb_stack_pass(int n_linears, const void* const* q, const void* const* meta, const void* const* s,
                              const int* k, const int* n, int n_widths, const int* width,
                              const void* const* x_of_width, void* const* xs_of_width, void* const* y_of, void* y_last,
                              const void* ids, int rows, int num_deltas, void* checksum, int groupsize, void* scratch,
                              size_t scratch_bytes, int dev, void* stream_v) {
  using namespace trb;
  if (n_linears <= 0 || rows <= 0) return TRB_OK;
  if (!q || !meta || !s || !k || !n || !width || !x_of_width || !xs_of_width || !y_of || !y_last || !ids || !checksum ||
      n_widths <= 0 || num_deltas <= 0)
    return TRB_ERR_BAD_ARG;
  if (!scratch || ((uintptr_t)scratch & 255) || scratch_bytes < trb_stack_scratch_bytes(rows, num_deltas)) return TRB_ERR_SCRATCH;
  if (groupsize != -1 && groupsize != 128) return TRB_ERR_KERN_SHAPE;
  for (int i = 0; i < n_linears; ++i) {
    if (k[i] % 128 != 0 || n[i] % 128 != 0 || k[i] <= 0 || n[i] <= 0) return TRB_ERR_PROB_SHAPE;
    bool found = false;
    for (int w = 0; w < n_widths; ++w) found = found || width[w] == k[i];
    if (!found) return TRB_ERR_BAD_ARG;
  }
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  cudaStream_t stream = (cudaStream_t)stream_v;

  const bool use_big = rows > kBigMinTokens;
  const size_t cap_small = small_tile_capacity(rows, num_deltas), cap_big = big_tile_capacity(rows);
  uint8_t* p = (uint8_t*)scratch;
  int* counters = (int*)p; p += kCounterBytes;
  int* perm = (int*)p; p += align_up((size_t)rows * 4, 256);
  RouteList small{}, big{};
  auto carve = [&](RouteList& l, size_t cap) {
    l.tile_delta = (int*)p; p += align_up(cap * 4, 256);
    l.tile_start = (int*)p; p += align_up(cap * 4, 256);
    l.tile_count = (int*)p; p += align_up(cap * 4, 256);
  };
  carve(small, cap_small);
  carve(big, cap_big);
  float* ksplit_buf = (float*)p;
  RouteClasses cl{};
  cl.small_max = kSmallSegMax;
  cl.tt_big = kBigTile;
  cl.big = big;
  RouteSrc src{};
  src.indices = (const int*)ids;
  int r = route_launch_src(src, rows, num_deltas, kSmallTile, perm, nullptr, nullptr, nullptr, small.tile_delta,
                           small.tile_start, small.tile_count, counters, nullptr, 0, nullptr, stream, use_big ? &cl : nullptr);
  if (r != TRB_OK) return r;
  for (int w = 0; w < n_widths; ++w) {
    // the first gather also clears the rows of y_last whose id selects no delta
    r = gather_launch(x_of_width[w], perm, counters, xs_of_width[w], w == 0 ? y_last : nullptr, rows, width[w],
                      n[n_linears - 1], w == 0 ? 1 : 0, stream, w == 0 ? counters + kKsplitCntOffset : nullptr, kKsplitItems);
    if (r != TRB_OK) return r;
  }
  for (int i = 0; i < n_linears; ++i) {
    const bool last = i == n_linears - 1;
    const void* xs = nullptr;
    for (int w = 0; w < n_widths; ++w)
      if (width[w] == k[i]) xs = xs_of_width[w];
    void* y = last ? y_last : y_of[i];
    if (!q[i] || !meta[i] || !s[i] || !xs || !y) return TRB_ERR_BAD_ARG;
    GemmArgs a{};
    a.mode = kSegTiles;
    a.rows = rows; a.N = n[i]; a.K = k[i]; a.num_deltas = num_deltas;
    a.grouped = groupsize == 128;
    a.scales = (const __half*)s[i];
    a.y = (__half*)y;
    a.row_map = last ? perm : nullptr;       // the last output goes back to the caller's row order
    GemmCall c{xs, q[i], meta[i], s[i], num_deltas, groupsize, dev, -1, stream};
    if (use_big) {
      a.seg_delta = big.tile_delta; a.seg_start = big.tile_start; a.seg_count = big.tile_count;
      a.n_seg_ptr = counters + 4;
      a.n_seg = (int)cap_big;
      r = gemm_dispatch(c, a, kBigTile);
      if (r != TRB_OK) return r;
    }
    a.seg_delta = small.tile_delta; a.seg_start = small.tile_start; a.seg_count = small.tile_count;
    a.n_seg_ptr = counters + 1;
    a.n_seg = (int)cap_small;
    a.ksplit_cnt = counters + kKsplitCntOffset;
    a.ksplit_buf = ksplit_buf;
    r = gemm_dispatch(c, a, kSmallTile);
    if (r != TRB_OK) return r;
    r = row_checksum_launch(y, checksum, rows, n[i], 1, last ? nullptr : perm, last ? nullptr : counters + 2, stream);
    if (r != TRB_OK) return r;
  }
  return TRB_OK;
}
