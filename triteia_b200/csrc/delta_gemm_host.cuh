// Host side of the grouped 2:4-sparse delta GEMM: tensor-map construction, configuration choice
// and the C entry points that stand in for the reference's launchers
// (marlin_cuda_2_4, csrc/ops/marlin_nm.cu:42-119; triteia_cuda_sbmm_2_4,
// csrc/ops/triteia_nm_sbmm.cu:809-847; triteia_cuda_bmm_2_4, csrc/ops/triteia_nm_bmm.cu:760-834).
#include "delta_gemm.cuh"

#include <cudaTypedefs.h>
#include <atomic>
#include <mutex>

namespace trb {

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// 2-D row-major tensor [rows, cols] of `esize`-byte elements, box [box_rows, box_cols].
static bool make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int esize, const void* base, uint64_t rows,
                        uint64_t cols, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
  auto fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)esize};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sm_count(int dev) {
  static std::atomic<int> cached[64];
  if (dev < 0 || dev >= 64) return 148;
  int v = cached[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cached[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

// cudaFuncSetAttribute(max dynamic shared memory) once per device and kernel; safe from any host thread.
template <class Kernel>
static bool ensure_smem_attr(Kernel kernel, int dev, int bytes, std::atomic<bool>* done /* [64] */) {
  if (dev < 0 || dev >= 64) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
  if (done[dev].load(std::memory_order_acquire)) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  done[dev].store(true, std::memory_order_release);
  return true;
}

struct GemmCall {
  const void* x;
  const void* q;
  const void* meta;
  const void* s;
  int num_deltas, groupsize, dev, sms;
  cudaStream_t stream;
};

template <class Cfg>
static int launch_cfg(const GemmCall& c, const GemmArgs& a) {
  const int slabs = a.K / 32;
  const int groups = a.grouped ? a.K / 128 : 1;
  CUtensorMap tx, tq, tm, ts;
  if (!make_map_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, c.x, (uint64_t)a.rows, (uint64_t)a.K, Cfg::TT, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return TRB_ERR_CUDA;
  if (!make_map_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, c.q, (uint64_t)c.num_deltas * slabs, 2ull * a.N, Cfg::KS,
                   Cfg::QB * 128, CU_TENSOR_MAP_SWIZZLE_NONE))
    return TRB_ERR_CUDA;
  if (!make_map_2d(&tm, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, c.meta, (uint64_t)c.num_deltas * slabs, (uint64_t)a.N,
                   Cfg::KS, Cfg::QB * 64, CU_TENSOR_MAP_SWIZZLE_NONE))
    return TRB_ERR_CUDA;
  if (a.grouped) {
    if (!make_map_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, c.s, (uint64_t)c.num_deltas * groups, (uint64_t)a.N,
                     Cfg::KS / 4, Cfg::SB * 64, CU_TENSOR_MAP_SWIZZLE_NONE))
      return TRB_ERR_CUDA;
  } else {
    ts = tm;  // never dereferenced
  }
  static std::atomic<bool> attr_set[64];
  if (!ensure_smem_attr(delta_gemm_kernel<Cfg>, c.dev, Cfg::SMEM_ALLOC, attr_set)) return TRB_ERR_CUDA;
  int grid = sm_count(c.dev);
  if (c.sms > 0 && c.sms < grid) grid = c.sms;
  // Upper bound on work items known on the host: never launch more CTAs than that.
  const int n_stripes = (a.N + Cfg::SW * 64 - 1) / (Cfg::SW * 64);
  long long max_tiles;
  if (a.mode == kSegSingle) max_tiles = (a.rows + Cfg::TT - 1) / Cfg::TT;
  else if (a.mode == kSegIdentity) max_tiles = a.rows;
  else if (a.mode == kSegTiles) max_tiles = a.n_seg;
  else max_tiles = (long long)a.rows / Cfg::TT + a.n_seg;
  const long long max_items = max_tiles * n_stripes;
  // With the tail K split the idle CTAs of a small launch take pieces of the items: keep the full grid.
  if (max_items < grid && a.ksplit_buf == nullptr) grid = (int)(max_items > 0 ? max_items : 1);
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid);
  lc.blockDim = dim3(Cfg::THREADS);
  lc.dynamicSmemBytes = Cfg::SMEM_ALLOC;
  lc.stream = c.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits (pdl_wait) before it reads
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return cudaLaunchKernelEx(&lc, delta_gemm_kernel<Cfg>, tx, tq, tm, ts, a) == cudaSuccess ? TRB_OK
                                                                                                             : TRB_ERR_CUDA;
}

// Prefill-sized tiles: the sparse tcgen05 / TMEM kernel.
template <class Cfg, class Kernel>
static int launch_tc_impl(Kernel kernel, const GemmCall& c, const GemmArgs& a) {
  const int slabs = a.K / 32;
  const int groups = a.grouped ? a.K / 128 : 1;
  CUtensorMap tx, tq, tm, ts;
  if (!make_map_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, c.x, (uint64_t)a.rows, (uint64_t)a.K, Cfg::B_ROWS, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return TRB_ERR_CUDA;
  if (!make_map_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, c.q, (uint64_t)c.num_deltas * slabs, 2ull * a.N, 2, 256,
                   CU_TENSOR_MAP_SWIZZLE_NONE))
    return TRB_ERR_CUDA;
  if (!make_map_2d(&tm, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, c.meta, (uint64_t)c.num_deltas * slabs, (uint64_t)a.N, 2, 128,
                   CU_TENSOR_MAP_SWIZZLE_NONE))
    return TRB_ERR_CUDA;
  if (a.grouped) {
    if (!make_map_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, c.s, (uint64_t)c.num_deltas * groups, (uint64_t)a.N, 1, 128,
                     CU_TENSOR_MAP_SWIZZLE_NONE))
      return TRB_ERR_CUDA;
  } else {
    ts = tm;  // never dereferenced
  }
  static std::atomic<bool> attr_set[64];   // one per instantiation of this template, that is per kernel
  if (!ensure_smem_attr(kernel, c.dev, Cfg::SMEM_ALLOC, attr_set)) return TRB_ERR_CUDA;
  constexpr int ctas = Cfg::CTAS;
  int grid = sm_count(c.dev);
  if (c.sms > 0 && c.sms < grid) grid = c.sms;
  grid /= ctas;                      // work items go to CTAs, or to clusters of two
  if (grid < 1) grid = 1;
  const int n_stripes = (a.N + Cfg::SW * 64 - 1) / (Cfg::SW * 64);
  long long max_tiles;
  if (a.mode == kSegSingle) max_tiles = (a.rows + Cfg::TT - 1) / Cfg::TT;
  else if (a.mode == kSegIdentity) max_tiles = a.rows;
  else if (a.mode == kSegTiles) max_tiles = a.n_seg;
  else max_tiles = (long long)a.rows / Cfg::TT + a.n_seg;
  const long long max_items = max_tiles * n_stripes;
  if (max_items < grid) grid = (int)(max_items > 0 ? max_items : 1);
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid * ctas);
  lc.blockDim = dim3(Cfg::THREADS);
  lc.dynamicSmemBytes = Cfg::SMEM_ALLOC;
  lc.stream = c.stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = ctas;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernels wait (pdl_wait) before they read
  at[1].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 2;
  return cudaLaunchKernelEx(&lc, kernel, tx, tq, tm, ts, a) == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}
static int launch_tc(const GemmCall& c, const GemmArgs& a) {
  // The sparse kernel writes y in 16-byte pieces of 8 output features.
  if ((reinterpret_cast<uintptr_t>(a.y) & 15) != 0 || (a.N & 7) != 0) return TRB_ERR_KERN_SHAPE;
  return launch_tc_impl<TcSpPairCfg>(delta_gemm_tcsp_kernel<true>, c, a);
}
static_assert(TcSpPairCfg::SMEM_ALLOC <= 232448, "shared memory budget of one sm_100 CTA");

// The mma.sp kernel works on tiles of 8 tokens (decode: a delta has a handful of tokens).  Larger
// tile classes of the same kernel (16 and 32 tokens) were built and measured: compiled beside the
// 8-token path they cost its hot loop registers (86 -> 102 us on the decode benchmark), and as a
// kernel of their own they ran under-filled launches slower than either neighbour, so segments are
// cut into 8-token tiles up to kSmallSegMax tokens and go to the tcgen05 kernel beyond that.
// Wide outputs: 256-column items, two warps per column block (half as many work items, so half the
// per-item cost per byte streamed); otherwise 128-column items, four warps per column block.
using CfgWide8 = GemmCfg<1, 4, 2, 8, 5>;
using CfgNarrow8 = GemmCfg<1, 2, 4, 8, 6>;
static_assert(CfgWide8::SMEM_ALLOC <= 232448 && CfgNarrow8::SMEM_ALLOC <= 232448, "shared memory budget of one sm_100 CTA");
constexpr int kSmallTile = 8;      // token tile of the mma.sp kernel
constexpr int kBigTile = 256;      // token tile of the tcgen05 kernel
constexpr int kSmallSegMax = 32;   // the router sends segments of more tokens than this to the tcgen05 kernel ...
constexpr int kBigMinTokens = 128; // ... when the batch has more tokens than this (smaller batches: one launch)

int gemm_tile_tokens(int tokens_per_segment) { return tokens_per_segment <= kSmallSegMax ? kSmallTile : kBigTile; }

static int check_common(const void* A, const void* B, const void* meta, void* C, const void* s, int N, int T, int K,
                        int groupsize) {
  if (N < 0 || T < 0 || K < 0) return TRB_ERR_BAD_ARG;
  if (N == 0 || T == 0 || K == 0) return -1;  // nothing to do
  if (!A || !B || !meta || !C || !s) return TRB_ERR_BAD_ARG;
  if (N % 128 != 0 || K % 128 != 0) return TRB_ERR_PROB_SHAPE;
  if (groupsize != -1 && groupsize != 128) return TRB_ERR_KERN_SHAPE;
  const uintptr_t bits = (uintptr_t)A | (uintptr_t)B | (uintptr_t)meta | (uintptr_t)C | (uintptr_t)s;
  if (bits & 15) return TRB_ERR_BAD_ARG;
  return TRB_OK;
}

int gemm_dispatch(const GemmCall& c, const GemmArgs& a, int tile_tokens) {
  cudaError_t e = cudaSetDevice(c.dev);
  if (e != cudaSuccess) return TRB_ERR_CUDA;
  switch (tile_tokens) {
    case kSmallTile: return (a.N % 256 == 0 && a.N >= 2048) ? launch_cfg<CfgWide8>(c, a) : launch_cfg<CfgNarrow8>(c, a);
    case kBigTile: return a.y_peers ? TRB_ERR_KERN_SHAPE : launch_tc(c, a);
    default: return TRB_ERR_KERN_SHAPE;
  }
}

}  // namespace trb

using namespace trb;

extern "C" int trb_mul_2_4(const void* A, const void* B, const void* meta, void* C, const void* s, int prob_m,
                           int prob_n, int prob_k, void* workspace, int groupsize, int dev, void* stream,
                           int thread_k, int thread_m, int sms, int max_par) {
  (void)workspace; (void)thread_k; (void)thread_m; (void)max_par;
  const int rc = check_common(A, B, meta, C, s, prob_m, prob_n, prob_k, groupsize);
  if (rc == -1) return TRB_OK;
  if (rc != TRB_OK) return rc;
  GemmArgs a{};
  a.mode = kSegSingle;
  a.rows = prob_n; a.N = prob_m; a.K = prob_k; a.num_deltas = 1;
  a.grouped = groupsize == 128;
  a.scales = (const __half*)s;
  a.y = (__half*)C;
  GemmCall c{A, B, meta, s, 1, groupsize, dev, sms, (cudaStream_t)stream};
  return gemm_dispatch(c, a, gemm_tile_tokens(prob_n));
}

// trb_sbmm_2_4 with working memory for the small-tile kernel's tail K split: `ksplit` holds
// trb_sbmm_ksplit_bytes() bytes, 256-byte aligned, whose first 512 bytes are zero on entry (they
// are zero again when the launch has finished).  Without it (nullptr) this is trb_sbmm_2_4.
extern "C" size_t trb_sbmm_ksplit_bytes(void) { return 512 + kKsplitBufBytes; }

// tile_tokens: 0 = choose from the average segment length; kSmallTile / kBigTile = forced.
static int sbmm_segments(const void* A, const void* B, const void* meta, void* C, const void* s, const void* indices,
                         const void* starts, const void* counts, int prob_m, int prob_n, int prob_k, int prob_r,
                         int groupsize, int dev, void* stream, int sms, void* ksplit, size_t ksplit_bytes,
                         int tile_tokens = 0) {
  if (prob_r == 0) return TRB_OK;
  if (prob_r < 0 || !indices || !starts || !counts) return TRB_ERR_BAD_ARG;
  const int rc = check_common(A, B, meta, C, s, prob_m, prob_n, prob_k, groupsize);
  if (rc == -1) return TRB_OK;
  if (rc != TRB_OK) return rc;
  if (ksplit != nullptr && (((uintptr_t)ksplit & 255) != 0 || ksplit_bytes < trb_sbmm_ksplit_bytes())) return TRB_ERR_SCRATCH;
  GemmArgs a{};
  a.mode = kSegList;
  a.rows = prob_n; a.N = prob_m; a.K = prob_k;
  a.grouped = groupsize == 128;
  a.scales = (const __half*)s;
  a.y = (__half*)C;
  // The tensor maps need a row bound; the reference signature has no delta count, so the maps
  // cover the largest index space a 32-bit row coordinate allows and the ids are trusted as the
  // reference trusts them.
  const int slabs = prob_k / 32;
  const int max_d = (int)(((1ull << 31) - 1) / (uint64_t)slabs);
  GemmCall c{A, B, meta, s, max_d, groupsize, dev, sms, (cudaStream_t)stream};
  a.num_deltas = max_d;
  const int avg = (prob_n + prob_r - 1) / prob_r;
  const int tt = tile_tokens != 0 ? tile_tokens : gemm_tile_tokens(avg);
  // A launch takes at most kMaxSegments segments (its prefix table lives in shared memory): longer
  // lists go out in several launches, which write disjoint rows.  The tail K split needs the whole
  // list in one launch (its counters are per launch).
  for (int r0 = 0; r0 < prob_r; r0 += kMaxSegments) {
    a.seg_delta = (const int*)indices + r0; a.seg_start = (const int*)starts + r0; a.seg_count = (const int*)counts + r0;
    a.n_seg = prob_r - r0 < kMaxSegments ? prob_r - r0 : kMaxSegments;
    if (ksplit != nullptr && prob_r <= kMaxSegments) {
      a.ksplit_cnt = (int*)ksplit;
      a.ksplit_buf = (float*)((uint8_t*)ksplit + 512);
    }
    const int r = gemm_dispatch(c, a, tt);
    if (r != TRB_OK) return r;
  }
  return TRB_OK;
}

extern "C" int trb_sbmm_2_4_ksplit(const void* A, const void* B, const void* meta, void* C, const void* s,
                                   const void* indices, const void* starts, const void* counts, int prob_m,
                                   int prob_n, int prob_k, int prob_r, int groupsize, int dev, void* stream,
                                   void* ksplit, size_t ksplit_bytes) {
  return sbmm_segments(A, B, meta, C, s, indices, starts, counts, prob_m, prob_n, prob_k, prob_r, groupsize, dev,
                       stream, -1, ksplit, ksplit_bytes);
}

extern "C" int trb_sbmm_2_4(const void* A, const void* B, const void* meta, void* C, const void* s,
                            const void* indices, const void* starts, const void* counts, int prob_m, int prob_n,
                            int prob_k, int prob_r, void* workspace, int groupsize, int dev, void* stream,
                            int thread_k, int thread_m, int sms, int max_par) {
  (void)workspace; (void)thread_k; (void)thread_m; (void)max_par;
  return sbmm_segments(A, B, meta, C, s, indices, starts, counts, prob_m, prob_n, prob_k, prob_r, groupsize, dev,
                       stream, sms, nullptr, 0);
}

extern "C" int trb_bmm_2_4(const void* A, const void* B, const void* meta, void* C, const void* s, int prob_m,
                           int prob_n, int prob_k, void* workspace, int groupsize, int dev, void* stream,
                           int thread_k, int thread_m, int sms, int max_par) {
  (void)workspace; (void)thread_k; (void)thread_m; (void)max_par;
  const int rc = check_common(A, B, meta, C, s, prob_m, prob_n, prob_k, groupsize);
  if (rc == -1) return TRB_OK;
  if (rc != TRB_OK) return rc;
  GemmArgs a{};
  a.mode = kSegIdentity;
  a.rows = prob_n; a.N = prob_m; a.K = prob_k; a.num_deltas = prob_n;
  a.grouped = groupsize == 128;
  a.scales = (const __half*)s;
  a.y = (__half*)C;
  GemmCall c{A, B, meta, s, prob_n, groupsize, dev, sms, (cudaStream_t)stream};
  return gemm_dispatch(c, a, kSmallTile);
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Head of the indexed path's scratch: 64 ints of router counters, then the counters of the grouped
// kernel's tail K split.
constexpr size_t kCounterBytes = 1024;
constexpr int kKsplitCntOffset = 64;
static_assert(kKsplitCntOffset * 4 + kKsplitItems * 4 <= (int)kCounterBytes, "counters fit the scratch head");

// Capacity of the tile lists the router fills: 8-token tiles for segments of at most kSmallSegMax
// tokens (all segments in batches of at most kBigMinTokens tokens), kBigTile-token tiles for the rest.
static size_t small_tile_capacity(int num_tokens, int num_deltas) {
  return (size_t)trb_route_max_tiles(num_tokens, num_deltas, kSmallTile);
}
static size_t big_tile_capacity(int num_tokens) { return (size_t)(num_tokens / kBigTile + num_tokens / (kSmallSegMax + 1) + 1); }

// The least scratch the indexed path works with (no tail K split).
static size_t indexed_scratch_min(int num_tokens, int prob_k, int num_deltas) {
  if (num_tokens <= 0 || prob_k <= 0 || num_deltas <= 0) return kCounterBytes;
  size_t b = kCounterBytes;                                                      // counters
  b += align_up((size_t)num_tokens * 4, 256);                                    // perm
  b += 3 * align_up(small_tile_capacity(num_tokens, num_deltas) * 4, 256);       // tile list, short segments
  b += 3 * align_up(big_tile_capacity(num_tokens) * 4, 256);                     // tile list, long segments
  b += align_up((size_t)num_tokens * prob_k * 2, 256);                           // gathered activations
  return b;
}

extern "C" size_t trb_sbmm_indexed_scratch_min_bytes(int num_tokens, int prob_k, int num_deltas) {
  return indexed_scratch_min(num_tokens, prob_k, num_deltas);
}

// What the caller should provide: the minimum plus the partial-tile slots of the tail K split.
extern "C" size_t trb_sbmm_indexed_scratch_bytes(int num_tokens, int prob_k, int num_deltas) {
  return indexed_scratch_min(num_tokens, prob_k, num_deltas) + kKsplitBufBytes;
}

namespace trb {
// Router + row gather + grouped kernels.  `src` says where the ids come from; num_tokens counts the
// rows of x and y.  mode: 0 = overwrite rows that have a delta and zero the others, 1 = accumulate,
// 2 = overwrite rows that have a delta and leave the others untouched.
// The router cuts every segment into tiles that fit its own token count (the reference chooses its
// tile per delta the same way, triteia/csrc/ops/triteia_nm_sbmm.cu:756-762): segments of up to
// kSmallSegMax tokens -> 8-token tiles of the mma.sp kernel, longer ones -> 256-token tiles of the
// tcgen05 kernel.  The lists are consumed without the host knowing their lengths: a launch whose list
// is empty ends at once, and batches of at most kBigMinTokens tokens make the mma.sp launch only.
int sbmm_indexed_impl(const void* x, const void* qweights, const void* metas, const void* scales, const RouteSrc& src,
                      void* y, int num_tokens, int prob_m, int prob_k, int num_deltas, int groupsize, int mode,
                      void* scratch, size_t scratch_bytes, int dev, cudaStream_t stream,
                      const void* y_peers = nullptr, int chunk_rows = 0, int phases = 3) {
  // phases: bit 0 = router + gather (they write the scratch only, unless mode 0 zeroes rows of y),
  // bit 1 = the grouped kernels (they read the scratch and write y).
  if (num_deltas <= 0 || (phases & 3) == 0) return TRB_ERR_BAD_ARG;
  const int rc = check_common(x, qweights, metas, y, scales, prob_m, num_tokens, prob_k, groupsize);
  if (rc == -1) return TRB_OK;
  if (rc != TRB_OK) return rc;
  if (!scratch || ((uintptr_t)scratch & 255)) return TRB_ERR_BAD_ARG;
  const size_t min_bytes = indexed_scratch_min(num_tokens, prob_k, num_deltas);
  if (scratch_bytes < min_bytes) return TRB_ERR_SCRATCH;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;

  // The peer-store epilogue exists in the mma.sp kernel only; the tcgen05 kernel writes 16-byte pieces.
  const bool use_big = y_peers == nullptr && num_tokens > kBigMinTokens && (prob_m & 7) == 0;
  const size_t cap_small = small_tile_capacity(num_tokens, num_deltas), cap_big = big_tile_capacity(num_tokens);

  uint8_t* p = (uint8_t*)scratch;
  int* counters = (int*)p; p += kCounterBytes;
  // Tail K split of the mma.sp kernel: only with room for its partial tiles behind the rest.
  const bool ksplit = scratch_bytes >= min_bytes + kKsplitBufBytes;
  int* perm = (int*)p; p += align_up((size_t)num_tokens * 4, 256);
  RouteList small{}, big{};
  auto carve = [&](RouteList& l, size_t cap) {
    l.tile_delta = (int*)p; p += align_up(cap * 4, 256);
    l.tile_start = (int*)p; p += align_up(cap * 4, 256);
    l.tile_count = (int*)p; p += align_up(cap * 4, 256);
  };
  carve(small, cap_small);
  carve(big, cap_big);
  void* x_sorted = p;
  RouteClasses cl{};
  cl.small_max = kSmallSegMax;
  cl.tt_big = kBigTile;
  cl.big = big;

  int r = TRB_OK;
  if (phases & 1) {
    r = route_launch_src(src, num_tokens, num_deltas, kSmallTile, perm, nullptr, nullptr, nullptr, small.tile_delta,
                         small.tile_start, small.tile_count, counters, nullptr, 0, nullptr, stream,
                         use_big ? &cl : nullptr);
    if (r != TRB_OK) return r;
    r = gather_launch(x, perm, counters, x_sorted, y, num_tokens, prob_k, prob_m, mode == 0 ? 1 : 0, stream,
                      ksplit ? counters + kKsplitCntOffset : nullptr, kKsplitItems);
    if (r != TRB_OK) return r;
  }
  if (!(phases & 2)) return TRB_OK;

  GemmArgs a{};
  a.mode = kSegTiles;
  a.rows = num_tokens; a.N = prob_m; a.K = prob_k; a.num_deltas = num_deltas;
  a.grouped = groupsize == 128;
  a.scales = (const __half*)scales;
  a.y = (__half*)y;
  a.row_map = perm;
  a.accumulate = mode == 1;
  GemmCall c{x_sorted, qweights, metas, scales, num_deltas, groupsize, dev, -1, stream};
  if (use_big) {
    a.seg_delta = big.tile_delta; a.seg_start = big.tile_start; a.seg_count = big.tile_count;
    a.n_seg_ptr = counters + 4;
    a.n_seg = (int)cap_big;
    r = gemm_dispatch(c, a, kBigTile);
    if (r != TRB_OK) return r;
  }
  a.y_peers = (__half* const*)y_peers;
  a.xchg = src.chunk_base;
  a.xchg_row_bytes = src.row_bytes;
  a.chunk_rows = chunk_rows;
  a.seg_delta = small.tile_delta; a.seg_start = small.tile_start; a.seg_count = small.tile_count;
  a.n_seg_ptr = counters + 1;
  a.n_seg = (int)cap_small;
  if (ksplit) {
    a.ksplit_cnt = counters + kKsplitCntOffset;
    a.ksplit_buf = (float*)((uint8_t*)scratch + min_bytes);
  }
  return gemm_dispatch(c, a, kSmallTile);
}
}  // namespace trb

extern "C" int trb_sbmm_indexed(const void* x, const void* qweights, const void* metas, const void* scales,
                                const void* indices, void* y, int num_tokens, int prob_m, int prob_k,
                                int num_deltas, int index_offset, int groupsize, int accumulate, void* scratch,
                                size_t scratch_bytes, int dev, void* stream_v) {
  if (num_tokens > 0 && !indices) return TRB_ERR_BAD_ARG;
  RouteSrc src{};
  src.indices = (const int*)indices;
  src.id_offset = index_offset;
  return sbmm_indexed_impl(x, qweights, metas, scales, src, y, num_tokens, prob_m, prob_k, num_deltas, groupsize,
                           accumulate ? 1 : 0, scratch, scratch_bytes, dev, (cudaStream_t)stream_v);
}

// trb_sbmm_indexed in two calls, so that a caller can run the router and the row gather (phase 1:
// they touch nothing but the scratch when accumulate != 0) on one stream beside other work -- the
// base product of ldmm -- and the grouped kernels (phase 2) after both.  Same arguments and the
// same scratch in both calls; phase 3 = trb_sbmm_indexed.
extern "C" int trb_sbmm_indexed_phase(const void* x, const void* qweights, const void* metas, const void* scales,
                                      const void* indices, void* y, int num_tokens, int prob_m, int prob_k,
                                      int num_deltas, int index_offset, int groupsize, int accumulate, void* scratch,
                                      size_t scratch_bytes, int phase, int dev, void* stream_v) {
  if (num_tokens > 0 && !indices) return TRB_ERR_BAD_ARG;
  if (phase < 1 || phase > 3) return TRB_ERR_BAD_ARG;
  RouteSrc src{};
  src.indices = (const int*)indices;
  src.id_offset = index_offset;
  return sbmm_indexed_impl(x, qweights, metas, scales, src, y, num_tokens, prob_m, prob_k, num_deltas, groupsize,
                           accumulate ? 1 : 0, scratch, scratch_bytes, dev, (cudaStream_t)stream_v, nullptr, 0, phase);
}

// Owner-side step of the sharded path: the received exchange buffer (world chunks of cap + 1 rows of K
// halves, ids in each chunk's last row) goes through the router and the grouped kernel.  Plain form:
// result rows land in the same slots of `y_work` (world * (cap + 1) rows of N halves), other rows are
// left alone.  Peer form (peer_out_ptrs != NULL): every result row is stored into its source rank's
// output tensor [cap, N] at the token's own row, y_work is not used.
extern "C" int trb_shard_compute(const void* recv_buf, const void* qweights, const void* metas, const void* scales,
                                 void* y_work, int world, int cap, int prob_m, int prob_k, int num_local_deltas,
                                 int groupsize, const void* peer_out_ptrs, int my_rank, void* scratch,
                                 size_t scratch_bytes, int dev, void* stream_v) {
  (void)my_rank;
  if (world < 1 || cap < 1 || !recv_buf || (!y_work && !peer_out_ptrs)) return TRB_ERR_BAD_ARG;
  // The id row of a chunk holds cap ids and the row count (plain form), plus cap token rows (peer form).
  if ((long long)(cap + 1) * 4 > (long long)prob_k * 2) return TRB_ERR_PROB_SHAPE;
  if (peer_out_ptrs && ((long long)(2 * cap + 2) * 4 > (long long)prob_k * 2 || cap >= (1 << 20))) return TRB_ERR_PROB_SHAPE;
  const long long rows = (long long)world * (cap + 1);
  if (rows > 65536) return TRB_ERR_PROB_SHAPE;
  RouteSrc src{};
  src.chunk_base = (const unsigned char*)recv_buf;
  src.cap = cap;
  src.row_bytes = (long long)prob_k * 2;
  return sbmm_indexed_impl(recv_buf, qweights, metas, scales, src, y_work ? y_work : (void*)recv_buf, (int)rows, prob_m, prob_k, num_local_deltas,
                           groupsize, 2, scratch, scratch_bytes, dev, (cudaStream_t)stream_v, peer_out_ptrs, cap + 1);
}

extern "C" int trb_route(const void* indices, int num_tokens, int num_deltas, int tile_tokens, int index_offset,
                         void* perm,
                         void* seg_delta, void* seg_start, void* seg_count, void* tile_delta, void* tile_start,
                         void* tile_count, void* counters, int dev, void* stream) {
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  return route_launch((const int*)indices, num_tokens, num_deltas, tile_tokens, index_offset, (int*)perm, (int*)seg_delta,
                      (int*)seg_start, (int*)seg_count, (int*)tile_delta, (int*)tile_start, (int*)tile_count,
                      (int*)counters, (cudaStream_t)stream);
}

extern "C" int trb_device_status(int dev, int* status_out) {
  if (!status_out) return TRB_ERR_BAD_ARG;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  if (cudaDeviceSynchronize() != cudaSuccess) return TRB_ERR_CUDA;
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return TRB_ERR_CUDA;
  const int zero = 0;
  if (cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)) != cudaSuccess) return TRB_ERR_CUDA;
  *status_out = v;
  return TRB_OK;
}

// Self-test of the bounded waits: one CTA waits on an mbarrier that nothing ever signals, with a
// limit of `max_polls` polls.  The wait gives up by construction, the kernel records
// TRB_ERR_TIMEOUT in the device error word and ends normally; nothing hangs and the context stays
// usable.  trb_device_status then returns (and clears) the code.
namespace trb {
__global__ void selftest_timeout_kernel(uint32_t max_polls, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int dead;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    dead = 0;
    fence_mbar_init();
  }
  __syncthreads();
  mbar_wait(&bar, 0, &dead, max_polls);     // phase 0 never completes: no arrival is ever made
  __syncthreads();
  if (threadIdx.x == 0 && gave_up != nullptr) *gave_up = dead;
}
}  // namespace trb

extern "C" int trb_selftest_timeout(int max_polls, void* gave_up_flag, int dev, void* stream) {
  if (max_polls < 1 || max_polls > 1000000) return TRB_ERR_BAD_ARG;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  trb::selftest_timeout_kernel<<<1, 64, 0, (cudaStream_t)stream>>>((uint32_t)max_polls, (int*)gave_up_flag);
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}

extern "C" int trb_version(void) { return 101; }

extern "C" const char* trb_status_string(int status) {
  switch (status) {
    case TRB_OK: return "ok";
    case TRB_ERR_PROB_SHAPE: return "problem shape not supported";
    case TRB_ERR_KERN_SHAPE: return "no kernel implementation for this configuration";
    case TRB_ERR_BAD_ARG: return "bad argument (null or misaligned pointer, negative size)";
    case TRB_ERR_CUDA: return "CUDA call failed";
    case TRB_ERR_TIMEOUT: return "a bounded device-side wait expired";
    case TRB_ERR_SCRATCH: return "scratch buffer too small";
    default: return "unknown status";
  }
}
