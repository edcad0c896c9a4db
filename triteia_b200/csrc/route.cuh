// Token router: stable grouping of tokens by delta id (-1 first) and the tile work list, in one
// single-CTA launch with no host synchronisation.  Replaces the torch prologue of the reference
// (triteia/python/ops/matmul/sbmm.py:94-123: unique_consecutive, where, cumsum, three host
// syncs), and drops its requirement that the caller pre-sorts the indices.
//
// Counting sort made stable with warp-level primitives: the token range is cut into one
// contiguous piece per warp; each warp histograms its piece (match_any groups equal ids inside
// a 32-token step), a block-wide exclusive scan over (id-major, warp-minor) counts gives every
// (id, warp) pair its first output slot, and a second pass ranks tokens inside each step with
// match_any + popc.  All integer work; results are bit-exact against the CPU router.
#pragma once
#include <atomic>

#include "common.cuh"

namespace trb {

constexpr int kRouteThreads = 1024;   // upper bound; small batches launch 256

// Exclusive scan of data[0..len) in shared memory by the whole CTA; returns the total.
__device__ int block_exclusive_scan(int* data, int len, int* warp_tot /* [33] */) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nthreads = blockDim.x, nwarps = nthreads >> 5;
  const int per = (len + nthreads - 1) / nthreads;
  const int lo = min(len, tid * per), hi = min(len, lo + per);
  int sum = 0;
  for (int i = lo; i < hi; ++i) sum += data[i];
  int inc = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += v;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < nwarps ? warp_tot[lane] : 0;
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += v;
    }
    warp_tot[lane] = winc - w;
    if (lane == 31) warp_tot[32] = winc;
  }
  __syncthreads();
  int run = warp_tot[warp] + inc - sum;
  for (int i = lo; i < hi; ++i) {
    const int v = data[i];
    data[i] = run;
    run += v;
  }
  const int total = warp_tot[32];
  __syncthreads();
  return total;
}

// Where the ids come from and how an id becomes a bin.
struct RouteSrc {
  const int* indices;    // plain mode: one id per token
  int id_offset;         // id = raw - id_offset
  int mod;               // > 0: bin by id % mod (planning the dispatch to `mod` ranks)
  // Chunked mode (chunk_base != nullptr): token t is row t % (cap + 1) of chunk t / (cap + 1) of an
  // exchange buffer whose chunks are cap + 1 rows of row_bytes; the last row of a chunk holds the ids
  // of its rows as int32 followed by the number of rows in use.
  const unsigned char* chunk_base;
  int cap;
  long long row_bytes;
};

__device__ __forceinline__ int route_load_raw(const RouteSrc& s, int t) {
  if (s.chunk_base == nullptr) return s.indices[t];
  const int rows = s.cap + 1;
  const int r = t / rows, q = t - r * rows;
  if (q == s.cap) return -1;
  const int* ids = reinterpret_cast<const int*>(s.chunk_base + ((long long)r * rows + s.cap) * s.row_bytes);
  return q < ids[s.cap] ? ids[q] : -1;
}

__device__ __forceinline__ int route_bin(const RouteSrc& s, int raw, int D, bool* invalid) {
  const int id = raw - s.id_offset;
  *invalid = raw < -1 || (s.mod <= 0 && id >= D);
  if (id < 0) return 0;
  if (s.mod > 0) return id % s.mod + 1;
  return id >= D ? 0 : id + 1;
}

// Tile lists by segment size.  With small_max > 0 a segment of more than small_max tokens leaves the
// first list (tiles of TT tokens) and is cut into tiles of tt_big tokens in the `big` list, so that
// short and long segments each get the kernel that suits them (the reference picks its tile per delta
// from the delta's token count, triteia/csrc/ops/triteia_nm_sbmm.cu:756-762).  counters[4] = length
// of the big list.
struct RouteList {
  int* tile_delta;
  int* tile_start;
  int* tile_count;
};
struct RouteClasses {
  int small_max, tt_big;
  RouteList big;
};

__global__ void __launch_bounds__(kRouteThreads, 1)
route_kernel(const RouteSrc src, int T, int D, int W, int TT, int* __restrict__ perm,
             int* __restrict__ seg_delta, int* __restrict__ seg_start, int* __restrict__ seg_count,
             int* __restrict__ tile_delta, int* __restrict__ tile_start, int* __restrict__ tile_count,
             int* __restrict__ counters, int* __restrict__ slot_of, int slot_stride, int* __restrict__ bin_count,
             const RouteClasses cl) {
  extern __shared__ int sm[];
  pdl_launch_dependents();
  const int bins = D + 1;             // bin 0 = id -1 (and out-of-range ids)
  int* hist = sm;                     // [bins][W]
  int* bin_start = hist + bins * W;   // [bins + 1]
  int* seg_flag = bin_start + bins + 1;   // [bins]
  int* tile_cnt = seg_flag + bins;        // [bins]
  int* tile_cnt2 = tile_cnt + bins;       // [bins] tiles in the big list
  __shared__ int warp_tot[33];
  __shared__ int n_invalid;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < bins * W; i += blockDim.x) hist[i] = 0;
  if (tid == 0) n_invalid = 0;
  __syncthreads();
  // Launched with programmatic stream serialization: everything above overlaps the tail of the kernel
  // before; the ids may come from it and the outputs may still be read by it, so wait here.
  pdl_wait();

  const int piece = ((T + W - 1) / W + 31) / 32 * 32;   // tokens per warp, multiple of 32
  const int t_lo = warp * piece, t_hi = min(T, t_lo + piece);

  if (warp < W) {
    for (int base = t_lo; base < t_hi; base += 32) {
      const int t = base + lane;
      int bin = -1;
      if (t < t_hi) {
        bool bad;
        bin = route_bin(src, route_load_raw(src, t), D, &bad);
        if (bad) atomicAdd(&n_invalid, 1);
      }
      const unsigned active = __ballot_sync(0xffffffffu, bin >= 0);
      if (bin >= 0) {
        const unsigned same = __match_any_sync(active, bin);
        if ((same & ((1u << lane) - 1)) == 0) hist[bin * W + warp] += __popc(same);
      }
    }
  }
  __syncthreads();
  block_exclusive_scan(hist, bins * W, warp_tot);
  for (int b = tid; b < bins; b += blockDim.x) bin_start[b] = hist[b * W];
  if (tid == 0) bin_start[bins] = T;
  __syncthreads();

  if ((perm != nullptr || slot_of != nullptr) && warp < W) {
    for (int base = t_lo; base < t_hi; base += 32) {
      const int t = base + lane;
      int bin = -1;
      if (t < t_hi) {
        bool bad;
        bin = route_bin(src, route_load_raw(src, t), D, &bad);
      }
      const unsigned active = __ballot_sync(0xffffffffu, bin >= 0);
      if (bin >= 0) {
        const unsigned same = __match_any_sync(active, bin);
        const int rank = __popc(same & ((1u << lane) - 1));
        const int first = hist[bin * W + warp];
        __syncwarp(active);
        if (rank == 0) hist[bin * W + warp] = first + __popc(same);
        if (perm) perm[first + rank] = t;
        // Slot of the token inside its bin (dispatch planning): bin b - 1 owns slots
        // [(b - 1) * slot_stride, ...); tokens of bin 0 get -1.
        if (slot_of) slot_of[t] = bin == 0 ? -1 : (bin - 1) * slot_stride + (first + rank - bin_start[bin]);
      }
      __syncwarp();
    }
  }
  __syncthreads();

  // Segments (distinct ids >= 0 in increasing order) and their tiles.
  for (int b = tid; b < bins; b += blockDim.x) {
    const int cnt = bin_start[b + 1] - bin_start[b];
    const bool is_seg = b >= 1 && cnt > 0;
    const bool is_big = is_seg && cl.small_max > 0 && cnt > cl.small_max;
    seg_flag[b] = is_seg ? 1 : 0;
    tile_cnt[b] = (is_seg && !is_big) ? (cnt + TT - 1) / TT : 0;
    tile_cnt2[b] = is_big ? (cnt + cl.tt_big - 1) / cl.tt_big : 0;
  }
  __syncthreads();
  const int n_seg = block_exclusive_scan(seg_flag, bins, warp_tot);
  const int n_tiles = block_exclusive_scan(tile_cnt, bins, warp_tot);
  const int n_tiles2 = cl.small_max > 0 ? block_exclusive_scan(tile_cnt2, bins, warp_tot) : 0;
  for (int b = tid + 1; b < bins; b += blockDim.x) {
    const int start = bin_start[b], cnt = bin_start[b + 1] - start;
    if (cnt > 0) {
      const int s = seg_flag[b];
      if (seg_delta) seg_delta[s] = b - 1;
      if (seg_start) seg_start[s] = start;
      if (seg_count) seg_count[s] = cnt;
      if (cl.small_max > 0 && cnt > cl.small_max) {
        int tpos = tile_cnt2[b];
        for (int off = 0; off < cnt; off += cl.tt_big, ++tpos) {
          cl.big.tile_delta[tpos] = b - 1;
          cl.big.tile_start[tpos] = start + off;
          cl.big.tile_count[tpos] = min(cl.tt_big, cnt - off);
        }
      } else if (tile_delta && tile_start && tile_count) {
        int tpos = tile_cnt[b];
        for (int off = 0; off < cnt; off += TT, ++tpos) {
          tile_delta[tpos] = b - 1;
          tile_start[tpos] = start + off;
          tile_count[tpos] = min(TT, cnt - off);
        }
      }
    }
  }
  if (bin_count)
    for (int b = tid + 1; b < bins; b += blockDim.x) bin_count[b - 1] = bin_start[b + 1] - bin_start[b];
  if (tid == 0 && counters) {
    counters[0] = n_seg;
    counters[1] = n_tiles;
    counters[2] = bin_start[1];
    counters[3] = n_invalid;
    counters[4] = n_tiles2;
  }
}

// x_sorted[p] = x[perm[p]] for every sorted position; optionally zero y rows whose id is -1.
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ perm,
                                   const int* __restrict__ counters, uint4* __restrict__ x_sorted,
                                   uint4* __restrict__ y, int T, int k_vec, int n_vec, int zero_base_rows,
                                   int* __restrict__ zero_ints, int n_zero_ints) {
  const int p = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();                          // perm and counters come from the router launched just before
  // Counters of the grouped kernel's tail K split: zero at every call (the scratch is the caller's).
  if (p == 0 && zero_ints != nullptr)
    for (int i = threadIdx.x; i < n_zero_ints; i += blockDim.x) zero_ints[i] = 0;
  if (p >= T) return;
  const int src = perm[p];
  if (src < 0 || src >= T) return;
  const int n_neg = counters[2];
  if (p >= n_neg) {
    const uint4* s = x + (size_t)src * k_vec;
    uint4* d = x_sorted + (size_t)p * k_vec;
    for (int i = threadIdx.x; i < k_vec; i += blockDim.x) d[i] = s[i];
  } else if (zero_base_rows) {
    uint4* d = y + (size_t)src * n_vec;
    for (int i = threadIdx.x; i < n_vec; i += blockDim.x) d[i] = make_uint4(0, 0, 0, 0);
  }
}

}  // namespace trb

using namespace trb;

extern "C" int trb_route_max_tiles(int num_tokens, int num_deltas, int tile_tokens) {
  if (num_tokens <= 0 || tile_tokens <= 0) return 0;
  const int segs = num_tokens < num_deltas ? num_tokens : num_deltas;
  return num_tokens / tile_tokens + segs;
}

namespace trb {
int route_launch_src(const RouteSrc& src, int T, int D, int TT, int* perm, int* seg_delta, int* seg_start,
                     int* seg_count, int* tile_delta, int* tile_start, int* tile_count, int* counters, int* slot_of,
                     int slot_stride, int* bin_count, cudaStream_t stream, const RouteClasses* classes = nullptr) {
  if (T < 0 || T > 65536 || D < 1 || D > 8191 || TT < 1) return TRB_ERR_PROB_SHAPE;
  if ((src.indices == nullptr && src.chunk_base == nullptr && T > 0) || counters == nullptr) return TRB_ERR_BAD_ARG;
  const int bins = D + 1;
  // Small batches: 8 warps (cheaper block syncs), and no more histogram copies than 32-token pieces.
  // every warp should see at most one or two 32-token steps (each step is a chain of dependent loads)
  const int threads = (T <= 256 && bins <= 2048) ? 256 : kRouteThreads;
  int W = (50000 - 4 * bins - 1) / bins;   // shared-memory budget of ~195 KiB
  const int w_cap = threads / 32, w_need = (T + 31) / 32;
  W = W > w_cap ? w_cap : W;
  W = W > w_need ? w_need : W;
  W = W < 1 ? 1 : W;
  const size_t smem = (size_t)(bins * W + 4 * bins + 1) * sizeof(int);
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return TRB_ERR_CUDA;
    attr_set[dev].store(true, std::memory_order_release);
  }
  RouteClasses cl{};
  if (classes != nullptr) {
    cl = *classes;
    if (cl.small_max < 1 || cl.tt_big < 1 || !cl.big.tile_delta || !cl.big.tile_start || !cl.big.tile_count)
      return TRB_ERR_BAD_ARG;
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(1);
  lc.blockDim = dim3(threads);
  lc.dynamicSmemBytes = smem;
  lc.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits (pdl_wait) before its first global access
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return cudaLaunchKernelEx(&lc, route_kernel, src, T, D, W, TT, perm, seg_delta, seg_start, seg_count, tile_delta,
                            tile_start, tile_count, counters, slot_of, slot_stride, bin_count, cl) == cudaSuccess
             ? TRB_OK
             : TRB_ERR_CUDA;
}

int route_launch(const int* indices, int T, int D, int TT, int id_offset, int* perm, int* seg_delta, int* seg_start,
                 int* seg_count, int* tile_delta, int* tile_start, int* tile_count, int* counters,
                 cudaStream_t stream) {
  RouteSrc src{};
  src.indices = indices;
  src.id_offset = id_offset;
  return route_launch_src(src, T, D, TT, perm, seg_delta, seg_start, seg_count, tile_delta, tile_start, tile_count,
                          counters, nullptr, 0, nullptr, stream);
}

int gather_launch(const void* x, const int* perm, const int* counters, void* x_sorted, void* y, int T, int K,
                  int N, int zero_base_rows, cudaStream_t stream, int* zero_ints = nullptr, int n_zero_ints = 0) {
  if (T == 0) return TRB_OK;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(T);
  lc.blockDim = dim3(128);
  lc.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return cudaLaunchKernelEx(&lc, gather_rows_kernel, (const uint4*)x, perm, counters, (uint4*)x_sorted, (uint4*)y, T,
                            K / 8, N / 8, zero_base_rows, zero_ints, n_zero_ints) == cudaSuccess
             ? TRB_OK
             : TRB_ERR_CUDA;
}
}  // namespace trb
