// Grouped 2:4-sparse int4 delta GEMM for prefill-sized token tiles on the SPARSE fifth-generation
// tensor-core instruction: tcgen05.mma.sp (kind::f16, K = 32 dense per instruction), A operand = the
// STORED halves of the 2:4 weights in shared memory (16 per row and instruction), 2:4 metadata in
// tensor memory, fp32 accumulator in tensor memory.
//
// Forms of the kernel template:
//   PAIR (shipped)  two CTAs of a cluster issue one tcgen05.mma.sp.cta_group::2 per instruction:
//                   M = 256 output features (128 per CTA: each CTA decodes its own stripe and holds its
//                   own accumulator and metadata) x N = 256 tokens (each CTA stages 128 of them).  The
//                   leader CTA's MMA thread issues for both; every decode warp of both CTAs arrives on
//                   the leader's barrier; tcgen05.commit with a CTA mask hands stages back to both.
//                   Half the activation bytes per SM and flop: the kernel is bound by what one SM can
//                   pull through TMA and shared memory, not by the tensor pipe.
//   single CTA      M = 128 x N = 256 per CTA (PAIR = false; not instantiated in the library).
//
// Per 64-K chunk and per CTA:
//   producer warps  TMA, one thread each: the activation tile [tokens x 64 K] (128-byte swizzle, the B
//                   operand as it lands) / packed weights + metadata + scales of the CTA's 128 columns
//   16 decode warps two teams of eight on alternate chunks: nibbles -> fp16 (x group scale) stored as
//                   half2 pairs into the compressed A tile [128 features x 32 stored halves] (64-byte
//                   swizzle, K-major); the same warps copy the chunk's metadata into TMEM with
//                   tcgen05.st: the packed format already holds, per 32-K slab, one 16-bit field per
//                   row and K half in the tensor core's ordered 2-bit-index form, so a TMEM cell
//                   (lane = 16*(row/16) + 8*(K half) + row%8) is two such fields (rows r and r + 8)
//                   picked from two packed words with one PRMT
//   MMA warp        one thread issues 2 tcgen05.mma.sp per chunk; the metadata operand is the even
//                   column of the chunk's column pair, the instruction descriptor's id2 selects the
//                   slab; tcgen05.commit hands the stage back / publishes the tile
//   4 epilogue warps tcgen05.ld, scale, convert, transpose 32 x 32 blocks through shared memory and
//                   store 16-byte pieces (8 features of one token)
// TMEM: columns [0, 256) accumulator, [256, 256 + 2 * stages) metadata (a column pair per stage).
// Every wait is bounded; both CTAs of a pair meet at a cluster barrier before either leaves.
#pragma once

#include "tc_common.cuh"

namespace trb {

// PAIR: two CTAs of a cluster share one tcgen05.mma.sp.cta_group::2 (M = 256 features, 128 per CTA;
// each CTA stages half of the token tile), which halves the activation bytes every SM pulls through
// its shared memory per flop.
template <bool PAIR_>
struct TcSpCfgT {
  static constexpr bool PAIR = PAIR_;
  static constexpr int CTAS = PAIR ? 2 : 1;
  static constexpr int TT = 256;
  static constexpr int SW = 2 * CTAS;       // 64-column blocks per work item (128 columns per CTA)
  static constexpr int KC = 64;             // dense K per stage = two sparse MMAs
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr int B_ROWS = TT / CTAS;  // tokens of the tile staged by one CTA
  static constexpr int DECODE_TEAMS = 2;    // teams of 8 warps take alternate K chunks
  static constexpr int DECODE_WARPS = 8 * DECODE_TEAMS;
  static constexpr int EPI_WARPS = 8;       // two per TMEM lane quadrant: each drains half of the token batches
  static constexpr int THREADS = (3 + DECODE_WARPS + EPI_WARPS) * 32;
  static constexpr int A_BYTES = 128 * (KC / 2) * 2;     // 8 KiB of stored halves
  static constexpr int B_BYTES = B_ROWS * KC * 2;        // 32 KiB, 16 KiB per CTA of a pair
  static constexpr int Q_BYTES = 2 * 256 * 4;
  static constexpr int M_BYTES = 2 * 128 * 4;
  static constexpr int S_BYTES = 256;
  static constexpr int A_OFF = 0;
  static constexpr int B_OFF = A_OFF + A_BYTES;
  static constexpr int Q_OFF = B_OFF + B_BYTES;
  static constexpr int M_OFF = Q_OFF + Q_BYTES;
  static constexpr int S_OFF = M_OFF + M_BYTES;
  static constexpr int STAGE_BYTES = (S_OFF + S_BYTES + 1023) / 1024 * 1024;
  static constexpr int ROWS_OFF = STAGES * STAGE_BYTES;                   // int [TT] output rows
  static constexpr int XPOSE_OFF = ROWS_OFF + TT * 4;                     // [EPI_WARPS][32 tokens][32 features] halves
  static constexpr int PREFIX_OFF = XPOSE_OFF + EPI_WARPS * 2048;
  static constexpr int BAR_OFF = PREFIX_OFF + (kMaxSegments + 2) * 4;
  static constexpr int NUM_BARS = 3 * STAGES + 2;
  static constexpr int SMEM_BYTES = BAR_OFF + NUM_BARS * 8 + 16;
  static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t META_COL = 256;             // even: column pairs start on even columns
};
using TcSpCfg = TcSpCfgT<false>;
using TcSpPairCfg = TcSpCfgT<true>;

// K-major, 64-byte swizzle: rows of 64 bytes, 8-row groups 512 bytes apart, layout type 4.
__device__ __forceinline__ uint64_t tc_smem_desc_sw64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;
  return d;
}

// Sparse kind::f16: the dense descriptor plus the sparsity flag (bit 2) and the metadata id (bits 0-1).
__device__ __forceinline__ void tc_mma_sp_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t e_tmem,
                                              uint32_t id2, uint32_t accumulate) {
  const uint32_t idesc = kTcIdesc | (1u << 2) | (id2 & 3u);
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.sp.cta_group::1.kind::f16 [%0], %1, %2, [%9], %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u),
        "r"(e_tmem)
      : "memory");
}

__device__ __forceinline__ void tc_st1(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// ---- cluster-of-two helpers ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded like mbar_wait; observes arrivals made by the other CTA of the pair.
__device__ __forceinline__ void mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* dead) {
  uint32_t polls = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((polls & 15u) == 0 && *dead) return;
    if (++polls > kMaxPolls) {
      *dead = 1;
      atomicExch(&g_device_status, TRB_ERR_TIMEOUT);
      return;
    }
  }
}
// One instruction for both CTAs: M = 256 (128 TMEM lanes in each CTA), N = 256 tokens (128 rows of B
// from each CTA's shared memory), descriptors and TMEM addresses are CTA-relative and equal in both.
__device__ __forceinline__ void tc_mma_sp_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t e_tmem,
                                                   uint32_t id2, uint32_t accumulate) {
  constexpr uint32_t kIdesc = (1u << 4) | ((256u >> 3) << 17) | ((256u >> 4) << 24) | (1u << 2);
  const uint32_t idesc = kIdesc | (id2 & 3u);
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.sp.cta_group::2.kind::f16 [%0], %1, %2, [%6], %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(e_tmem)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs once the pair's MMAs issued so far retire.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}

template <bool PAIR>
__global__ void __launch_bounds__(TcSpCfgT<PAIR>::THREADS, 1)
delta_gemm_tcsp_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_q,
                       const __grid_constant__ CUtensorMap tm_m, const __grid_constant__ CUtensorMap tm_s,
                       const GemmArgs a) {
  using Cfg = TcSpCfgT<PAIR>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int* rows = reinterpret_cast<int*>(smem + Cfg::ROWS_OFF);
  int* prefix = reinterpret_cast<int*>(smem + Cfg::PREFIX_OFF);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);   // TMA data of a stage landed
  uint64_t* aready_bar = full_bar + STAGES;                                // A tile + metadata of a stage written
  uint64_t* empty_bar = aready_bar + STAGES;                               // MMAs of a stage retired
  uint64_t* accready_bar = empty_bar + STAGES;                             // accumulator complete
  uint64_t* accfree_bar = accready_bar + 1;                                // accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfree_bar + 1);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  int n_seg = 0;

  // A tile list that the router left empty (the usual case at decode sizes): leave before anything
  // is set up.  Both CTAs of a pair read the same count.
  pdl_launch_dependents();
  if (a.mode == kSegTiles && a.n_seg_ptr != nullptr) {
    pdl_wait();
    if (*a.n_seg_ptr <= 0) return;
  }

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&aready_bar[s], 8 * Cfg::CTAS);   // pair: the leader's barrier counts both CTAs' warps
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accready_bar, 1);
    mbar_init(accfree_bar, Cfg::EPI_WARPS * Cfg::CTAS);
    *dead = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(Cfg::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(Cfg::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  pdl_wait();   // everything below reads what the kernels launched before this one wrote
  n_seg = a.n_seg_ptr ? *a.n_seg_ptr : a.n_seg;
  n_seg = max(0, min(n_seg, a.mode == kSegTiles ? a.n_seg : kMaxSegments));
  int total_tiles;
  if (a.mode == kSegList) {
    if (warp == 0) {
      int running = 0;
      for (int base = 0; base < n_seg; base += 32) {
        const int s = base + lane;
        int c = 0;
        if (s < n_seg) {
          const int cnt = a.seg_count[s];
          c = cnt > 0 ? (cnt + Cfg::TT - 1) / Cfg::TT : 0;
        }
        int inc = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, inc, o);
          if (lane >= o) inc += v;
        }
        if (s < n_seg) prefix[s] = running + inc - c;
        running += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) prefix[n_seg] = running;
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();     // both CTAs' barriers exist before any remote arrive
  tc_fence_after();
  if (a.mode == kSegList) total_tiles = prefix[n_seg];
  else total_tiles = a.mode == kSegTiles ? n_seg : (a.mode == kSegSingle ? (a.rows + Cfg::TT - 1) / Cfg::TT : a.rows);
  const uint32_t tmem_base = *tmem_slot;

  const int n_stripes = (a.N + Cfg::SW * 64 - 1) / (Cfg::SW * 64);
  const int n_items = total_tiles * n_stripes;
  // Work items go round-robin over CTAs, or over CTA pairs: CTA `rank` of a pair owns columns
  // [col0 + 128 * rank, +128) of the item and stages tokens [row0 + 128 * rank, +128) of its tile.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int item0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int item_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int my_col = (int)rank * 128;
  const int slabs = a.K / 32;
  const int k_chunks = a.K / Cfg::KC;
  const int groups = a.grouped ? a.K / 128 : 1;
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0) {
    // ------------------------------ TMA producer: activations ------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_x);
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_m);
      if (a.grouped) prefetch_tmap(&tm_s);
      const uint64_t pol_x = policy_evict_last();
      const uint32_t stage_tx = Cfg::B_BYTES + Cfg::Q_BYTES + Cfg::M_BYTES + (a.grouped ? Cfg::S_BYTES : 0);
      int st = 0;
      uint32_t phase = 0;
      for (int item = item0; item < n_items; item += item_step) {
        WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, item);
        if (!w.ok) continue;
        for (int kc = 0; kc < k_chunks; ++kc) {
          mbar_wait(&empty_bar[st], phase ^ 1, dead);
          uint8_t* sbase = smem + st * Cfg::STAGE_BYTES;
          // The stage's one arrival, carrying the bytes of this load and of the weight producer's loads.
          mbar_arrive_expect_tx(&full_bar[st], stage_tx);
          tma_load_2d_hint(sbase + Cfg::B_OFF, &tm_x, kc * Cfg::KC, w.row0 + (int)rank * Cfg::B_ROWS, &full_bar[st], pol_x);
          if (++st == STAGES) { st = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && rank == 0) {
      int st = 0;
      uint32_t phase = 0, use = 0;
      for (int item = item0; item < n_items; item += item_step) {
        WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, item);
        w.col0 += my_col;
        if (!w.ok) continue;
        if constexpr (PAIR) mbar_wait_cluster(accfree_bar, (use & 1) ^ 1, dead);
        else mbar_wait(accfree_bar, (use & 1) ^ 1, dead);
        tc_fence_after();
        for (int kc = 0; kc < k_chunks; ++kc) {
          if constexpr (PAIR) {
            // Every decode warp of both CTAs arrives after its own CTA's TMA data landed and its part of
            // the A tile and metadata is written: the one barrier covers both CTAs' operands.
            mbar_wait_cluster(&aready_bar[st], phase, dead);
          } else {
            mbar_wait(&full_bar[st], phase, dead);
            mbar_wait(&aready_bar[st], phase, dead);
          }
          tc_fence_after();
          const uint32_t sb = smem_base + st * Cfg::STAGE_BYTES;
          const uint64_t adesc = tc_smem_desc_sw64(sb + Cfg::A_OFF);
          const uint64_t bdesc = tc_smem_desc(sb + Cfg::B_OFF);
          const uint32_t e_tmem = tmem_base + Cfg::META_COL + 2 * st;
#pragma unroll
          for (int k = 0; k < 2; ++k) {  // per instruction: 32 bytes of stored A, 64 bytes of B, metadata column k of the pair
            if constexpr (PAIR) tc_mma_sp_f16_pair(tmem_base, adesc + 2 * k, bdesc + 4 * k, e_tmem, k, (kc > 0 || k > 0) ? 1u : 0u);
            else tc_mma_sp_f16(tmem_base, adesc + 2 * k, bdesc + 4 * k, e_tmem, k, (kc > 0 || k > 0) ? 1u : 0u);
          }
          if constexpr (PAIR) tc_commit_pair(&empty_bar[st]);
          else tc_commit(&empty_bar[st]);
          if (++st == STAGES) { st = 0; phase ^= 1; }
        }
        if constexpr (PAIR) tc_commit_pair(accready_bar);
        else tc_commit(accready_bar);
        ++use;
      }
    }
  } else if (warp < 2 + Cfg::DECODE_WARPS) {
    // ------------------------------ decode warps: packed -> compressed A tile + metadata ------------------------------
    // Warp dw handles column block cb = dw / 4 and row groups g = 2 * (dw % 4) + u; lane bits are
    // (j high, slab s, lane-in-quad m, j low): it decodes weight word (s, cb, g, m, j) for u = 0, 1.
    const int team = (warp - 2) >> 3;
    const int dw = (warp - 2) & 7;
    const int cb = dw >> 2;
    const int s = (lane >> 3) & 1, m = (lane >> 1) & 3, j = ((lane >> 4) << 1) | (lane & 1);
    uint32_t q_off[2], s_off[2], st_off[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int g = 2 * (dw & 3) + u;
      q_off[u] = Cfg::Q_OFF + s * 1024 + cb * 512 + (4 * g + m) * 16 + j * 4;
      s_off[u] = Cfg::S_OFF + (cb * 64 + 8 * g + 2 * j) * 2;
      const int n0 = cb * 64 + 8 * g + j;            // block-0 row; block-1 row is n0 + 4
#pragma unroll
      for (int p = 0; p < 4; ++p) {                  // pairs: (n0, grp m), (n0, grp m+4), (n1, m), (n1, m+4)
        const int n = n0 + 4 * (p >> 1);
        const int kc4 = 8 * s + m + 4 * (p & 1);     // 4-byte pair index inside the 64-byte row (= K group of the chunk)
        st_off[u][p] = Cfg::A_OFF + (n >> 3) * 512 + (n & 7) * 64 + ((((kc4 >> 2) ^ ((n >> 1) & 3))) << 4) + (kc4 & 3) * 4;
      }
    }
    // Metadata duty: TMEM lanes of this warp's quadrant, slab ms of the chunk.  Lane L of the tile is
    // (row block L / 16, K half (L / 8) % 2, row L % 8): its cell is the 16-bit field of that K half for
    // rows r = 16 * (L / 16) + L % 8 (low) and r + 8 (high).  Row r of the stripe is column block r / 64,
    // group g = (r % 64) / 8, position r % 8 = j + 4 * hi: its field is the low (hi = 0) or high half of
    // metadata word 2 * (j & 1) + 32 * (j >> 1) + 4 * g + (K half) of that block; r + 8 is group g + 1.
    const int quad = warp & 3;
    const int ms = dw >> 2;
    const int L = quad * 32 + lane;
    const int mr = 16 * (L >> 4) + (L & 7);
    const int mk1 = (L >> 3) & 1;
    const int mj = mr & 3, mhi = (mr >> 2) & 1, mg = (mr & 63) >> 3;
    const uint32_t ma_off = Cfg::M_OFF + ms * 512 + ((mr >> 6) * 64 + 2 * (mj & 1) + 32 * (mj >> 1) + 4 * mg + mk1) * 4;
    const uint32_t msel = mhi ? 0x7632u : 0x5410u;
    const uint32_t e_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + Cfg::META_COL + ms;

    const uint32_t aready_leader = PAIR ? mapa_shared(smem_u32(aready_bar), 0) : 0u;
    int st = 0;
    uint32_t phase = 0, chunk = 0;
    for (int item = item0; item < n_items; item += item_step) {
      WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, item);
      w.col0 += my_col;
      if (!w.ok) continue;
      for (int kc = 0; kc < k_chunks; ++kc, ++chunk) {
        if ((int)(chunk % Cfg::DECODE_TEAMS) != team) {     // the other team's chunk
          if (++st == STAGES) { st = 0; phase ^= 1; }
          continue;
        }
        if (dw == 0) mbar_wait(&full_bar[st], phase, dead);   // one warp of the team polls
        named_bar_sync(5 + team, 256);
        const uint32_t sb = smem_base + st * Cfg::STAGE_BYTES;
        {
          const uint32_t wa = lds32(sb + ma_off), wb = lds32(sb + ma_off + 16);
          tc_st1(e_lane + 2 * st, __byte_perm(wa, wb, msel));
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t q = lds32(sb + q_off[u]);
          uint32_t v[4];
          int4x4_to_half2x2(q, v[0], v[1]);
          int4x4_to_half2x2(q >> 8, v[2], v[3]);
          if (a.grouped) {
            const uint32_t sc = lds32(sb + s_off[u]);  // (scale of n0, scale of n1)
            const uint32_t s0 = __byte_perm(sc, 0, 0x1010), s1 = __byte_perm(sc, 0, 0x3232);
            v[0] = hmul2_u32(v[0], s0); v[1] = hmul2_u32(v[1], s0);
            v[2] = hmul2_u32(v[2], s1); v[3] = hmul2_u32(v[3], s1);
          }
#pragma unroll
          for (int p = 0; p < 4; ++p) sts32(sb + st_off[u][p], v[p]);
        }
        tc_wait_st();
        fence_proxy_async();      // the tensor core reads the A tile through the async proxy
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(aready_leader + st * 8);
          else mbar_arrive(&aready_bar[st]);
        }
        if (++st == STAGES) { st = 0; phase ^= 1; }
      }
    }
  } else if (warp == 2 + Cfg::DECODE_WARPS + Cfg::EPI_WARPS) {
    // ------------------------------ TMA producer: packed weights, metadata, scales ------------------------------
    // A thread of its own: the TMA unit takes the small boxes while the activation box is in flight.
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first();
      int st = 0;
      uint32_t phase = 0;
      for (int item = item0; item < n_items; item += item_step) {
        WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, item);
        w.col0 += my_col;
        if (!w.ok) continue;
        for (int kc = 0; kc < k_chunks; ++kc) {
          mbar_wait(&empty_bar[st], phase ^ 1, dead);
          uint8_t* sbase = smem + st * Cfg::STAGE_BYTES;
          const int wrow = w.delta * slabs + kc * 2;
          tma_load_2d_hint(sbase + Cfg::Q_OFF, &tm_q, (w.col0 / 64) * 128, wrow, &full_bar[st], pol_w);
          tma_load_2d_hint(sbase + Cfg::M_OFF, &tm_m, (w.col0 / 64) * 64, wrow, &full_bar[st], pol_w);
          if (a.grouped)
            tma_load_2d_hint(sbase + Cfg::S_OFF, &tm_s, w.col0, w.delta * groups + kc / 2, &full_bar[st], pol_w);
          if (++st == STAGES) { st = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int ew = warp - 2 - Cfg::DECODE_WARPS;
    const int quad = warp & 3;
    uint32_t use = 0;
    for (int item = item0; item < n_items; item += item_step) {
      WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, item);
      w.col0 += my_col;
      if (!w.ok) continue;
      for (int t = ew * 32 + lane; t < Cfg::TT; t += Cfg::EPI_WARPS * 32) {
        int r = -1;
        if (t < w.valid) {
          r = w.row0 + t;
          if (a.row_map) r = a.row_map[r];
          if (r < 0 || r >= a.rows) r = -1;
        }
        rows[t] = r;
      }
      const int n = w.col0 + quad * 32 + lane;
      float sf = 1.f;
      if (!a.grouped && n < a.N) sf = __half2float(a.scales[(size_t)w.delta * a.N + n]);
      // One warp polls the barrier (a shared-memory access per poll), the others park on the
      // hardware barrier; the wait spans the whole K loop of the item, so the poller backs off.
      if (ew == 0) {
        uint32_t polls = 0;
        while (!mbar_try_wait(accready_bar, use & 1)) {
          __nanosleep(128);
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
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
      const int nbatch = max(1, (w.valid + 31) >> 5);
      // The two warps of a quadrant split the 32-token batches; each hands the accumulator back once,
      // when its last batch is in registers (at once if it has none): the next item's MMAs may then
      // overwrite it.
      const int per = (nbatch + 1) >> 1;
      const int b0 = (ew >> 2) * per, b1 = min(nbatch, b0 + per);
      auto release = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(accfree_bar), 0));
          else mbar_arrive(accfree_bar);
        }
      };
      if (b1 <= b0) release();
      for (int b = b0; b < b1; ++b) {
        uint32_t v[32];
        tc_ld32(taddr + b * 32, v);
        tc_wait_ld();
        if (b == b1 - 1) release();
        // Transpose the 32-token x 32-feature block through a private 2 KiB patch of shared memory, so
        // that a lane stores 8 consecutive features (16 bytes) of one token instead of one feature.
        {
          __half* patch = reinterpret_cast<__half*>(smem + Cfg::XPOSE_OFF + ew * 2048);
#pragma unroll
          for (int c = 0; c < 32; ++c) patch[c * 32 + lane] = __float2half_rn(__uint_as_float(v[c]) * sf);
          __syncwarp();
          const int f8 = (lane & 3) * 8;                    // feature offset of this lane's 16-byte piece
          const int nb = w.col0 + quad * 32 + f8;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int c = i * 8 + (lane >> 2);              // token of the batch
            const int r = rows[b * 32 + c];
            if (r >= 0 && nb < a.N) {
              uint4 o = *reinterpret_cast<const uint4*>(patch + c * 32 + f8);
              uint4* yp = reinterpret_cast<uint4*>(a.y + (size_t)r * a.N + nb);
              if (a.accumulate) {
                const uint4 old = *yp;
                __half2* oh = reinterpret_cast<__half2*>(&o);
                const __half2* ph = reinterpret_cast<const __half2*>(&old);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 x = __half22float2(oh[e]), y2 = __half22float2(ph[e]);
                  oh[e] = __floats2half2_rn(x.x + y2.x, x.y + y2.y);
                }
              }
              *yp = o;
            }
          }
          __syncwarp();
        }
      }
      named_bar_sync(4, Cfg::EPI_WARPS * 32);          // rows[] is rewritten for the next item after this
      ++use;
    }
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // neither CTA leaves, or frees TMEM, while the other may still touch it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
  }
}

}  // namespace trb
