// Dense fp16 base GEMM of the path, y[T, N] (+)= x[T, K] * W_base[N, K]^T, with the LoRA expand folded
// into the same accumulator: y += V[T, Kv] * B[Kv, N], where V holds every token's rank-r shrink
// result in the column block of its adapter (zero elsewhere) and B is the adapters' expand matrices
// stacked along K (the natural [M, r, N] tensor seen as [M * r, N]).
//
// The reference runs the base product as torch.matmul (a library GEMM) and then adds the LoRA and
// delta parts in separate passes over y (triteia/python/ops/matmul/ldmm.py:72-76, 86-107;
// sbmm.py:90-93; lora.py:5-9).  Here one kernel on the fifth-generation tensor cores produces
// base + LoRA in one TMEM accumulator and writes y once:
//   tcgen05.mma.cta_group::2.kind::f16: two CTAs of a cluster work on one item of 256 output features
//   x one token tile, 128 features each (own A tile, own accumulator: TMEM lanes = features, columns =
//   tokens) and each stages HALF of the token tile, so an SM pulls a third less through TMA per flop
//   than alone -- at 256 decode tokens the product is bound by that intake, not by the tensor pipe or
//   HBM; two accumulators, so the epilogue of one work item overlaps the MMAs of the next;
//   A operand = W_base rows [128 x 64 K] as they lie in memory (K-major, TMA with 128-byte swizzle),
//   for the LoRA chunks = B rows [64 Kv x 128 features] as they lie in memory (MN-major operand);
//   B operand = x (or V) rows [token tile x 64 K], K-major;
//   warp 0: TMA producer (one thread), warp 1: MMA issuer (one thread of the leader CTA) and TMEM
//   owner, warps 2-5: epilogue (tcgen05.ld, fp16 convert, 32 x 32 transposes through shared memory,
//   16-byte stores), warp 6: tells the leader when this CTA's stage has landed.  No TMA load uses
//   multicast.  Every wait is bounded; both CTAs meet at a cluster barrier before either leaves.
#pragma once

#include "delta_gemm_tcsp.cuh"

namespace trb {

struct BaseCfg {
  static constexpr int KC = 64;             // K per pipeline stage (one 128-byte swizzle atom of fp16)
  static constexpr int STAGES = 6;
  static constexpr int EPI_WARPS = 8;       // two per TMEM lane quadrant: each takes half of the token batches
  static constexpr int THREADS = (3 + EPI_WARPS) * 32;
  static constexpr int MAX_TT = 256;        // largest token tile (UMMA N)
  static constexpr int A_BYTES = 128 * KC * 2;                 // 16 KiB: this CTA's 128 features
  static constexpr int B_BYTES = (MAX_TT / 2) * KC * 2;        // 16 KiB: this CTA's half of the token tile
  static constexpr int A_OFF = 0;
  static constexpr int B_OFF = A_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;        // 32 KiB, a multiple of 1 KiB
  static constexpr int XPOSE_OFF = STAGES * STAGE_BYTES;                  // [EPI_WARPS][32 tokens][32 features] halves
  static constexpr int PREFIX_OFF = XPOSE_OFF + EPI_WARPS * 2048;         // int [kMaxSegments + 2]: tiles before each segment
  static constexpr int BAR_OFF = PREFIX_OFF + (kMaxSegments + 2) * 4;
  static constexpr int NUM_BARS = 3 * STAGES + 4;
  static constexpr int SMEM_BYTES = BAR_OFF + NUM_BARS * 8 + 16;
  static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = 512;
};
static_assert(BaseCfg::STAGE_BYTES % 1024 == 0, "stages keep the 1 KiB alignment of the swizzle atoms");

struct BaseArgs {
  int T, N, K;        // tokens, output features, input features (K % 64 == 0)
  int kv;             // K extent of the LoRA part (0: none); columns of V and rows of B
  int tt;             // token tile: 32, 64, 128 or 256
  __half* y;          // fp16 or bf16 by `bf16`
  int accumulate;     // y += result instead of y = result
  int bf16;           // operands and output are bfloat16
  // Segmented form (seg != nullptr), the SGMV of the LoRA operators: rows [seg[i], seg[i + 1]) of the
  // input [T, seg_k] meet weight i of a stacked tensor [n_seg, seg_k, N] (row-major, so an MN-major
  // operand as it lies in memory).  K is unused, x is the input, the stacked weights come through tm_b.
  const int* seg;
  int n_seg, seg_k;
};

// MN-major operand, 128-byte swizzle: a row of the tile is one K index and holds 64 consecutive
// M (feature) elements = 128 bytes; 8 K rows form a 1 KiB group (stride offset), the next 64
// features start `lbo` bytes further (leading offset).
__device__ __forceinline__ uint64_t tc_smem_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Dense kind::f16 for a CTA pair with a run-time instruction descriptor (token tile and operand
// majorness vary): M = 256 (128 TMEM lanes in each CTA), N rows of B split over the two CTAs.
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

__global__ void __launch_bounds__(BaseCfg::THREADS, 1)
base_gemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_b,
                 const BaseArgs a) {
  using Cfg = BaseCfg;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int* prefix = reinterpret_cast<int*>(smem + Cfg::PREFIX_OFF);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);   // this CTA's TMA data of a stage landed
  uint64_t* ready_bar = full_bar + STAGES;                                 // leader: both CTAs' data landed
  uint64_t* empty_bar = ready_bar + STAGES;                                // MMAs of a stage retired
  uint64_t* accready_bar = empty_bar + STAGES;                             // [2] accumulator complete
  uint64_t* accfree_bar = accready_bar + 2;                                // [2] leader: accumulator drained by both
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfree_bar + 2);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  pdl_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&ready_bar[s], 2);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&accready_bar[b], 1);
      mbar_init(&accfree_bar[b], 2 * Cfg::EPI_WARPS);   // every epilogue warp of both CTAs
    }
    *dead = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  pdl_wait();   // x and V may come from the kernels launched just before
  const int n_seg = a.seg != nullptr ? max(0, min(a.n_seg, kMaxSegments)) : 0;
  if (a.seg != nullptr && warp == 0) {   // token tiles before each segment
    int running = 0;
    for (int base = 0; base < n_seg; base += 32) {
      const int sg = base + lane;
      int c = 0;
      if (sg < n_seg) {
        const int cnt = a.seg[sg + 1] - max(0, a.seg[sg]);
        c = cnt > 0 ? (cnt + a.tt - 1) / a.tt : 0;
      }
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      if (sg < n_seg) prefix[sg] = running + inc - c;
      running += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) prefix[n_seg] = running;
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // both CTAs' barriers exist before any remote arrive
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t rank = cluster_ctarank();
  const int n_stripes = (a.N + 255) / 256;            // an item: 256 features (128 per CTA) x one token tile
  const int n_tiles = a.seg != nullptr ? prefix[n_seg] : (a.T + a.tt - 1) / a.tt;
  const int n_items = n_tiles * n_stripes;            // item = tile * n_stripes + stripe
  // Token tile -> (first row, rows in use, segment).
  auto tile_rows = [&](int tile, int& row0, int& valid, int& sg) {
    if (a.seg == nullptr) {
      sg = 0;
      row0 = tile * a.tt;
      valid = min(a.tt, a.T - row0);
      return;
    }
    int lo = 0, hi = n_seg;  // largest segment with prefix[seg] <= tile
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid] <= tile) lo = mid; else hi = mid;
    }
    sg = lo;
    const int start = max(0, a.seg[sg]), end = min(a.T, a.seg[sg + 1]);
    row0 = start + (tile - prefix[sg]) * a.tt;
    valid = max(0, min(a.tt, end - row0));
  };
  const int item0 = (int)(blockIdx.x >> 1), item_step = (int)(gridDim.x >> 1);
  const int half_tt = a.tt >> 1;                      // tokens of a tile staged by one CTA
  const int kw = a.seg != nullptr ? 0 : a.K / Cfg::KC;                                  // chunks of the base product
  const int kl = ((a.seg != nullptr ? a.seg_k : a.kv) + Cfg::KC - 1) / Cfg::KC;         // MN-major chunks (LoRA)
  const int k_chunks = kw + kl;
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_x);
      prefetch_tmap(&tm_w);
      if (kl > 0) {
        prefetch_tmap(&tm_v);
        prefetch_tmap(&tm_b);
      }
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      const uint32_t stage_tx = Cfg::A_BYTES + half_tt * Cfg::KC * 2;
      int st = 0;
      uint32_t phase = 0;
      for (int item = item0; item < n_items; item += item_step) {
        const int tile = item / n_stripes, stripe = item - tile * n_stripes;
        int row0, valid, sg;
        tile_rows(tile, row0, valid, sg);
        row0 += (int)rank * half_tt;
        const int col0 = stripe * 256 + (int)rank * 128;
        const int wrow0 = a.seg != nullptr ? sg * a.seg_k : 0;      // first row of this segment's weight
        const CUtensorMap* tm_in = a.seg != nullptr ? &tm_x : &tm_v;
        for (int kc = 0; kc < k_chunks; ++kc) {
          mbar_wait(&empty_bar[st], phase ^ 1, dead);
          uint8_t* sbase = smem + st * Cfg::STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[st], stage_tx);
          if (kc < kw) {
            tma_load_2d_hint(sbase + Cfg::A_OFF, &tm_w, kc * Cfg::KC, col0, &full_bar[st], pol_w);
            tma_load_2d_hint(sbase + Cfg::B_OFF, &tm_x, kc * Cfg::KC, row0, &full_bar[st], pol_x);
          } else {
            const int j = kc - kw;
            // two boxes of [64 K rows x 64 features]: features col0.. and col0 + 64..
            tma_load_2d_hint(sbase + Cfg::A_OFF, &tm_b, col0, wrow0 + j * Cfg::KC, &full_bar[st], pol_x);
            tma_load_2d_hint(sbase + Cfg::A_OFF + 8192, &tm_b, col0 + 64, wrow0 + j * Cfg::KC, &full_bar[st], pol_x);
            tma_load_2d_hint(sbase + Cfg::B_OFF, tm_in, j * Cfg::KC, row0, &full_bar[st], pol_x);
          }
          if (++st == STAGES) { st = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA) ------------------------------
    if (lane == 0 && rank == 0) {
      // D fp32, A and B fp16 / bf16; N = token tile, M = 256; bit 15: A is MN-major (the LoRA chunks)
      const uint32_t fmt = a.bf16 ? 1u : 0u;           // operand format field: 0 = fp16, 1 = bf16
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (((uint32_t)a.tt >> 3) << 17) | ((256u >> 4) << 24);
      const uint32_t idesc_mn = idesc | (1u << 15);
      int st = 0;
      uint32_t phase = 0;
      uint32_t use[2] = {0, 0};
      int local = 0;
      for (int item = item0; item < n_items; item += item_step) {
        const int buf = local & 1;
        mbar_wait_cluster(&accfree_bar[buf], (use[buf] & 1) ^ 1, dead);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * Cfg::MAX_TT;
        for (int kc = 0; kc < k_chunks; ++kc) {
          mbar_wait_cluster(&ready_bar[st], phase, dead);
          tc_fence_after();
          const uint32_t sb = smem_base + st * Cfg::STAGE_BYTES;
          const uint64_t bdesc = tc_smem_desc(sb + Cfg::B_OFF);
          if (kc < kw) {
            const uint64_t adesc = tc_smem_desc(sb + Cfg::A_OFF);
#pragma unroll
            for (int k = 0; k < Cfg::KC / 16; ++k)   // +32 bytes of K per instruction = +2 in the address field
              tc_mma_f16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kc > 0 || k > 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int k = 0; k < Cfg::KC / 16; ++k) {  // 16 K rows of 128 bytes per instruction
              // 64-feature halves 8 KiB apart, 8-row K groups 1 KiB apart
              const uint64_t adesc = tc_smem_desc_mn(sb + Cfg::A_OFF + k * 2048, 8192, 1024);
              tc_mma_f16_pair(d_tmem, adesc, bdesc + 2 * k, idesc_mn, (kc > 0 || k > 0) ? 1u : 0u);
            }
          }
          tc_commit_pair(&empty_bar[st]);
          if (++st == STAGES) { st = 0; phase ^= 1; }
        }
        tc_commit_pair(&accready_bar[buf]);
        ++use[buf];
        ++local;
      }
    }
  } else if (warp == 2 + Cfg::EPI_WARPS) {
    // ------------------------------ stage relay: this CTA's data landed -> the leader ------------------------------
    if (lane == 0) {
      const uint32_t ready_leader = mapa_shared(smem_u32(ready_bar), 0);
      int st = 0;
      uint32_t phase = 0;
      for (int item = item0; item < n_items; item += item_step) {
        for (int kc = 0; kc < k_chunks; ++kc) {
          mbar_wait(&full_bar[st], phase, dead);
          mbar_arrive_cluster(ready_leader + st * 8);
          if (++st == STAGES) { st = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int ew = warp - 2;
    const int quad = warp & 3;                        // TMEM lanes this warp may touch: 32 * quad .. + 31
    const uint32_t accfree_leader = mapa_shared(smem_u32(accfree_bar), 0);
    uint32_t use[2] = {0, 0};
    int local = 0;
    for (int item = item0; item < n_items; item += item_step) {
      const int tile = item / n_stripes, stripe = item - tile * n_stripes;
      int row0, valid, sg;
      tile_rows(tile, row0, valid, sg);
      const int col0 = stripe * 256 + (int)rank * 128;
      const int buf = local & 1;
      // Each warp drains the 32-token batches b0, b0 + 1, ... of its TMEM lane quadrant (two warps share a
      // quadrant and split the batches).  Accumulating into y: the old values of all its batches are
      // fetched before the accumulator is complete, so the epilogue never waits on a load it just issued.
      constexpr int MAXB = BaseCfg::MAX_TT / 32 / 2;    // batches per warp
      const int f8 = (lane & 3) * 8;                  // feature offset of this lane's 16-byte piece
      const int nb = col0 + quad * 32 + f8;
      const int nbatch = max(1, (valid + 31) >> 5);
      const int per = (nbatch + 1) >> 1;
      const int b0 = (ew >> 2) * per, b1 = min(nbatch, b0 + per);
      auto piece = [&](int b, int i) -> uint4* {      // 16 bytes of token b * 32 + i * 8 + lane / 4, or nullptr
        const int t = b * 32 + i * 8 + (lane >> 2);
        return (t < valid && nb < a.N) ? reinterpret_cast<uint4*>(a.y + (size_t)(row0 + t) * a.N + nb) : nullptr;
      };
      uint4 old[MAXB][4];
      if (a.accumulate) {
#pragma unroll
        for (int k = 0; k < MAXB; ++k)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4* yp = b0 + k < b1 ? piece(b0 + k, i) : nullptr;
            old[k][i] = yp ? *yp : make_uint4(0, 0, 0, 0);
          }
      }
      if (ew == 0) {                                  // one warp polls, the others park on the hardware barrier
        uint32_t polls = 0;
        while (!mbar_try_wait(&accready_bar[buf], use[buf] & 1)) {
          __nanosleep(64);
          if ((polls & 15u) == 0 && *dead) break;
          if (++polls > kMaxPolls) {
            *dead = 1;
            atomicExch(&g_device_status, TRB_ERR_TIMEOUT);
            break;
          }
        }
      }
      named_bar_sync(4, Cfg::EPI_WARPS * 32);
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * Cfg::MAX_TT;
#pragma unroll
      for (int k = 0; k < MAXB; ++k) {
        const int b = b0 + k;
        uint32_t v[32];
        if (b < b1) {
          tc_ld32(taddr + b * 32, v);
          tc_wait_ld();
        }
        // hand the buffer back once per warp and item: after its last batch is in registers, or at
        // once if it has no batch
        if (b == b1 - 1 || (b1 <= b0 && k == 0)) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(accfree_leader + buf * 8);
        }
        if (b >= b1) continue;
        __half* patch = reinterpret_cast<__half*>(smem + Cfg::XPOSE_OFF + ew * 2048);
        if (a.bf16) {
          __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(patch);
#pragma unroll
          for (int c = 0; c < 32; ++c) pb[c * 32 + lane] = __float2bfloat16_rn(__uint_as_float(v[c]));
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) patch[c * 32 + lane] = __float2half_rn(__uint_as_float(v[c]));
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = i * 8 + (lane >> 2);          // token of the batch
          uint4* yp = piece(b, i);
          if (yp != nullptr) {
            uint4 o = *reinterpret_cast<const uint4*>(patch + c * 32 + f8);
            if (a.accumulate) {
              if (a.bf16) {
                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
                const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&old[k][i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 p = __bfloat1622float2(oh[e]), q = __bfloat1622float2(ph[e]);
                  oh[e] = __floats2bfloat162_rn(p.x + q.x, p.y + q.y);
                }
              } else {
                __half2* oh = reinterpret_cast<__half2*>(&o);
                const __half2* ph = reinterpret_cast<const __half2*>(&old[k][i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 p = __half22float2(oh[e]), q = __half22float2(ph[e]);
                  oh[e] = __floats2half2_rn(p.x + q.x, p.y + q.y);
                }
              }
            }
            *yp = o;
          }
        }
        __syncwarp();
      }
      ++use[buf];
      ++local;
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves, or frees TMEM, while the other may still touch it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
  }
}

// V[t, :] = 0 except columns [id * rank, (id + 1) * rank) = scale * x[t] @ A[id], for id = indices[t]
// in [0, num_adapters); the row stays zero for any other id.  One CTA per token, A [M, h1, rank] in
// its natural layout.  This is the shrink half of the reference's BGMV pair
// (triteia/csrc/ops/bgmv_impl.cuh:15-137) writing straight into the operand of the expand above.
constexpr int kShrinkThreads = 512;

template <class IdxT>
__global__ void __launch_bounds__(kShrinkThreads) lora_shrink_rows_kernel(__half* __restrict__ V, const __half* __restrict__ X,
                                                               const __half* __restrict__ A,
                                                               const IdxT* __restrict__ indices, int h1, int rank,
                                                               int num_adapters, int v_cols, float scale) {
  constexpr int WARPS = kShrinkThreads / 32;
  __shared__ float part[WARPS][64];
  const int b = blockIdx.x;
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint4* vrow = reinterpret_cast<uint4*>(V + (int64_t)b * v_cols);
  const long long idx = (long long)indices[b];
  const bool has = idx >= 0 && idx < num_adapters;
  const int lo8 = has ? (int)idx * rank / 8 : -1, hi8 = has ? lo8 + rank / 8 : -1;
  for (int i = tid; i < v_cols / 8; i += kShrinkThreads)
    if (i < lo8 || i >= hi8) vrow[i] = make_uint4(0, 0, 0, 0);
  if (!has) return;
  const __half* am = A + idx * (int64_t)h1 * rank;
  const __half* x = X + (int64_t)b * h1;
  // A row of A holds rank halves = rv 16-byte pieces.  `pw` lanes (rv rounded up to a power of two)
  // share a row, so a warp load covers 32 / pw consecutive rows: contiguous memory, 8 accumulators
  // per lane.
  const int rv = rank / 8;
  const int pw = rv <= 1 ? 1 : (rv <= 2 ? 2 : (rv <= 4 ? 4 : 8));
  const int sub = lane & (pw - 1), rl = lane / pw, rows_per_warp = 32 / pw;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  if (sub < rv) {
#pragma unroll 8
    for (int k = warp * rows_per_warp + rl; k < h1; k += WARPS * rows_per_warp) {
      const float xk = __half2float(x[k]);
      const uint4 wv = *reinterpret_cast<const uint4*>(am + (int64_t)k * rank + sub * 8);
      const uint32_t* pwv = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pwv[e]));
        acc[2 * e] = fmaf(xk, f.x, acc[2 * e]);
        acc[2 * e + 1] = fmaf(xk, f.y, acc[2 * e + 1]);
      }
    }
  }
  // lanes with the same `sub` hold partial sums of the same 8 columns
  for (int o = pw; o < 32; o <<= 1)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
  if (lane < pw && sub < rv)
#pragma unroll
    for (int e = 0; e < 8; ++e) part[warp][sub * 8 + e] = acc[e];
  __syncthreads();
  if (tid < rank) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) s += part[w][tid];
    V[(int64_t)b * v_cols + idx * rank + tid] = __float2half_rn(s * scale);
  }
}

static_assert(BaseCfg::SMEM_ALLOC <= 232448, "shared memory budget of one sm_100 CTA");

static int base_gemm_launch_args(const BaseArgs& a, const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& tv,
                                 const CUtensorMap& tb, long long items, int dev, cudaStream_t stream) {
  static std::atomic<bool> attr_set[64];
  if (!ensure_smem_attr(base_gemm_kernel, dev, BaseCfg::SMEM_ALLOC, attr_set)) return TRB_ERR_CUDA;
  int pairs = sm_count(dev) / 2;
  if (pairs < 1) pairs = 1;
  if (items < pairs) pairs = (int)(items > 0 ? items : 1);
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(2 * pairs);
  lc.blockDim = dim3(BaseCfg::THREADS);
  lc.dynamicSmemBytes = BaseCfg::SMEM_ALLOC;
  lc.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits (pdl_wait) before it reads
  at[0].val.programmaticStreamSerializationAllowed = 1;
  at[1].id = cudaLaunchAttributeClusterDimension;
  at[1].val.clusterDim.x = 2;
  at[1].val.clusterDim.y = 1;
  at[1].val.clusterDim.z = 1;
  lc.attrs = at;
  lc.numAttrs = 2;
  return cudaLaunchKernelEx(&lc, base_gemm_kernel, tx, tw, tv, tb, a) == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}

static int token_tile_for(int rows) { return rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : 256; }

static int base_gemm_launch(const void* x, const void* w, void* y, int T, int N, int K, const void* v, const void* b,
                            int kv, int accumulate, int bf16, int dev, cudaStream_t stream) {
  BaseArgs a{};
  a.T = T; a.N = N; a.K = K; a.kv = kv;
  a.tt = token_tile_for(T);
  a.y = (__half*)y;
  a.accumulate = accumulate;
  a.bf16 = bf16;
  const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tx, tw, tv, tb;
  if (!make_map_2d(&tx, dt, 2, x, (uint64_t)T, (uint64_t)K, a.tt / 2, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return TRB_ERR_CUDA;
  if (!make_map_2d(&tw, dt, 2, w, (uint64_t)N, (uint64_t)K, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return TRB_ERR_CUDA;
  if (kv > 0) {
    if (!make_map_2d(&tv, dt, 2, v, (uint64_t)T, (uint64_t)kv, a.tt / 2, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return TRB_ERR_CUDA;
    if (!make_map_2d(&tb, dt, 2, b, (uint64_t)kv, (uint64_t)N, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return TRB_ERR_CUDA;
  } else {
    tv = tx;   // never dereferenced
    tb = tw;
  }
  const long long items = (long long)((T + a.tt - 1) / a.tt) * ((N + 255) / 256);   // one item per CTA pair
  return base_gemm_launch_args(a, tx, tw, tv, tb, items, dev, stream);
}

// Segmented form: y[seg[i] : seg[i + 1]] (+)= x[same rows] @ w[i], w stacked [n_seg, d_in, d_out].
static int sgmv_stacked_launch(void* y, const void* x, const void* w, const int* seg, int n_seg, int T, int d_in,
                               int d_out, int max_rows, int accumulate, int bf16, int dev, cudaStream_t stream) {
  BaseArgs a{};
  a.T = T; a.N = d_out; a.K = 0; a.kv = 0;
  a.tt = token_tile_for(max_rows > 0 ? max_rows : T);
  a.y = (__half*)y;
  a.accumulate = accumulate;
  a.bf16 = bf16;
  a.seg = seg; a.n_seg = n_seg; a.seg_k = d_in;
  const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tx, tb;
  if (!make_map_2d(&tx, dt, 2, x, (uint64_t)T, (uint64_t)d_in, a.tt / 2, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return TRB_ERR_CUDA;
  if (!make_map_2d(&tb, dt, 2, w, (uint64_t)n_seg * d_in, (uint64_t)d_out, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return TRB_ERR_CUDA;
  const long long items = ((long long)T / a.tt + n_seg) * ((d_out + 255) / 256);     // upper bound: the lengths are on the device
  return base_gemm_launch_args(a, tx, tx, tx, tb, items, dev, stream);
}

}  // namespace trb

extern "C" int trb_base_gemm(const void* x, const void* base_weight, void* y, int num_tokens, int prob_m, int prob_k,
                             const void* lora_v, const void* lora_b, int lora_k, int accumulate, int dtype, int dev,
                             void* stream) {
  using namespace trb;
  if (num_tokens < 0 || prob_m < 0 || prob_k < 0 || lora_k < 0) return TRB_ERR_BAD_ARG;
  if (num_tokens == 0 || prob_m == 0) return TRB_OK;
  if (!x || !base_weight || !y || (lora_k > 0 && (!lora_v || !lora_b))) return TRB_ERR_BAD_ARG;
  if (prob_k == 0 || prob_k % 64 != 0 || prob_m % 8 != 0 || lora_k % 8 != 0) return TRB_ERR_PROB_SHAPE;
  if (dtype != TRB_F16 && dtype != TRB_BF16) return TRB_ERR_KERN_SHAPE;
  const uintptr_t bits = (uintptr_t)x | (uintptr_t)base_weight | (uintptr_t)y | (uintptr_t)lora_v | (uintptr_t)lora_b;
  if (bits & 15) return TRB_ERR_BAD_ARG;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  return base_gemm_launch(x, base_weight, y, num_tokens, prob_m, prob_k, lora_v, lora_b, lora_k, accumulate ? 1 : 0,
                          dtype == TRB_BF16, dev, (cudaStream_t)stream);
}

extern "C" int trb_sgmv_stacked(void* y, const void* x, const void* w, const void* s, int num_problems, int num_rows,
                                int d_in, int d_out, int max_rows, int accumulate, int dtype, int dev, void* stream) {
  using namespace trb;
  if (num_problems == 0 || num_rows == 0) return TRB_OK;
  if (num_problems < 0 || num_rows < 0 || !y || !x || !w || !s) return TRB_ERR_BAD_ARG;
  if (d_in <= 0 || d_out <= 0 || d_in % 8 != 0 || d_out % 8 != 0 || num_problems > kMaxSegments) return TRB_ERR_KERN_SHAPE;
  if ((long long)num_problems * d_in >= (1ll << 31)) return TRB_ERR_KERN_SHAPE;
  if (dtype != TRB_F16 && dtype != TRB_BF16) return TRB_ERR_KERN_SHAPE;
  if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)w) & 15) return TRB_ERR_BAD_ARG;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  return sgmv_stacked_launch(y, x, w, (const int*)s, num_problems, num_rows, d_in, d_out, max_rows, accumulate ? 1 : 0,
                             dtype == TRB_BF16, dev, (cudaStream_t)stream);
}

extern "C" int trb_lora_shrink_rows(void* v, const void* x, const void* wa, const void* indices, int index_is_64bit,
                                    int batch, int h1, int rank, int num_adapters, int v_cols, float scale, int dev,
                                    void* stream) {
  using namespace trb;
  if (batch == 0) return TRB_OK;
  if (batch < 0 || num_adapters <= 0 || !v || !x || !wa || !indices) return TRB_ERR_BAD_ARG;
  if (rank <= 0 || rank > 64 || rank % 8 != 0 || h1 <= 0 || v_cols % 8 != 0 || (long long)num_adapters * rank > v_cols)
    return TRB_ERR_KERN_SHAPE;
  if (((uintptr_t)v | (uintptr_t)wa) & 15) return TRB_ERR_BAD_ARG;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  cudaStream_t st = (cudaStream_t)stream;
  if (index_is_64bit)
    lora_shrink_rows_kernel<int64_t><<<batch, kShrinkThreads, 0, st>>>((__half*)v, (const __half*)x, (const __half*)wa,
                                                            (const int64_t*)indices, h1, rank, num_adapters, v_cols, scale);
  else
    lora_shrink_rows_kernel<int32_t><<<batch, kShrinkThreads, 0, st>>>((__half*)v, (const __half*)x, (const __half*)wa,
                                                            (const int32_t*)indices, h1, rank, num_adapters, v_cols, scale);
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}
