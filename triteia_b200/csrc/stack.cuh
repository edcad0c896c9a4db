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
                                    int accumulate) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
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
  if (lane == 0) sums[warp] = accumulate ? sums[warp] + acc : acc;
}

}  // namespace trb

extern "C" int trb_row_checksum(const void* y, void* sums, int rows, int prob_m, int accumulate, int dev,
                                void* stream) {
  using namespace trb;
  if (rows <= 0) return TRB_OK;
  if (!y || !sums) return TRB_ERR_BAD_ARG;
  if (prob_m <= 0 || prob_m % 8 != 0 || (reinterpret_cast<uintptr_t>(y) & 15) != 0) return TRB_ERR_PROB_SHAPE;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3((rows + 7) / 8);
  lc.blockDim = dim3(256);
  lc.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits before it reads y
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return cudaLaunchKernelEx(&lc, row_checksum_kernel, (const uint4*)y, (float*)sums, rows, prob_m / 8,
                            accumulate) == cudaSuccess
             ? TRB_OK
             : TRB_ERR_CUDA;
}

// One pass of a stack of independent delta linears over grouped rows, issued from C so that the
// host cost per launch is a few microseconds (a Python call per launch costs more than most of
// these kernels run).  Rows are grouped by (segment size class, delta id); every class is a
// contiguous row range with its own segment list and gets its own launch per linear, so the
// grouped kernel that fits the class runs (class_tile[c]: 8 = the mma.sp kernel, 256 = the tcgen05 kernel).  `ksplit` (optional): working memory
// of trb_sbmm_ksplit_bytes() bytes for the tail K split of small launches, first 512 bytes zero on
// entry (and again on exit).  After each linear its output is
// folded into the per-row checksum.  Arrays are host arrays; the pointers in them are device
// pointers.  x_of[i] / y_of[i]: grouped activations [rows, k[i]] and output buffer [rows, n[i]]
// of linear i (outputs of the same width may share a buffer: the checksum is taken before the
// next linear overwrites it).  No counterpart in the reference.
extern "C" int trb_stack_pass(int n_linears, const void* const* q, const void* const* meta, const void* const* s,
                              const int* k, const int* n, const void* const* x_of, void* const* y_of,
                              int n_classes, const int* class_row0, const int* class_rows,
                              const void* const* class_ids, const void* const* class_starts,
                              const void* const* class_counts, const int* class_segs, const int* class_tile,
                              void* checksum, int rows, int groupsize, void* ksplit, size_t ksplit_bytes, int dev,
                              void* stream) {
  if (n_linears <= 0 || rows <= 0) return TRB_OK;
  if (!q || !meta || !s || !k || !n || !x_of || !y_of || !checksum) return TRB_ERR_BAD_ARG;
  if (n_classes < 0 || (n_classes > 0 && (!class_row0 || !class_rows || !class_ids || !class_starts ||
                                          !class_counts || !class_segs || !class_tile)))
    return TRB_ERR_BAD_ARG;
  for (int c = 0; c < n_classes; ++c)
    if (class_row0[c] < 0 || class_rows[c] < 0 || class_row0[c] + class_rows[c] > rows) return TRB_ERR_BAD_ARG;
  for (int i = 0; i < n_linears; ++i) {
    for (int c = 0; c < n_classes; ++c) {
      if (class_rows[c] == 0 || class_segs[c] == 0) continue;
      const __half* x = (const __half*)x_of[i] + (size_t)class_row0[c] * k[i];
      __half* y = (__half*)y_of[i] + (size_t)class_row0[c] * n[i];
      if (class_tile[c] != trb::kSmallTile && class_tile[c] != trb::kBigTile) return TRB_ERR_BAD_ARG;
      const bool small = class_tile[c] == trb::kSmallTile;
      const int rc = sbmm_segments(x, q[i], meta[i], y, s[i], class_ids[c], class_starts[c], class_counts[c], n[i],
                                   class_rows[c], k[i], class_segs[c], groupsize, dev, stream, -1,
                                   small ? ksplit : nullptr, small ? ksplit_bytes : 0, class_tile[c]);
      if (rc != TRB_OK) return rc;
    }
    const int rc = trb_row_checksum(y_of[i], checksum, rows, n[i], 1, dev, stream);
    if (rc != TRB_OK) return rc;
  }
  return TRB_OK;
}
