// Grouped 2:4-sparse int4 delta GEMM for prefill-sized token tiles (tensor-bound regime) on the
// fifth-generation tensor cores: tcgen05.mma (kind::f16, M = 128 output features x N = 256 tokens
// x K = 16 per instruction) with the fp32 accumulator in tensor memory (TMEM).
//
// Per 64-K chunk and per CTA:
//   producer warp   TMA: packed weights + metadata + scales of a 128-column stripe, and the
//                   activation tile [256 tokens x 64 K] (128-byte swizzle = the tensor core's
//                   canonical K-major layout, used as the B operand as it lands)
//   8 decode warps  nibbles -> fp16 (x group scale), 2:4 metadata -> positions, each group of four K
//                   positions assembled in registers and stored as one 8-byte piece into the A
//                   operand tile [128 features x 64 K] in the same canonical swizzled layout
//   MMA warp        one thread issues 4 tcgen05.mma per chunk (A and B from shared memory through
//                   matrix descriptors), tcgen05.commit hands the stage back / publishes the tile
//   4 epilogue warps tcgen05.ld the accumulator (TMEM lane = output feature, column = token), scale,
//                   convert, store 32 consecutive features of one token per warp instruction
// The accumulator is double-buffered in TMEM (2 x 256 columns), so the epilogue of one work item
// overlaps the MMAs of the next.  The weights are the A operand (Y^T = W X^T): the packed format keeps
// the two stored values of every 2:4 group in one register pair, which is what makes the in-register
// re-layout cheap.  Format references as in delta_gemm.cuh.
#pragma once

#include "delta_gemm.cuh"

namespace trb {

struct TcCfg {
  static constexpr int TT = 256;            // tokens per tile (UMMA N)
  static constexpr int B_ROWS = TT;         // tokens staged by one CTA
  static constexpr int SW = 2;              // 64-column blocks per stripe (UMMA M = 128)
  static constexpr int CTAS = 1;
  static constexpr int KC = 64;             // dense K per pipeline stage (one 128-byte swizzle atom)
  static constexpr int STAGES = 4;
  static constexpr int DECODE_WARPS = 16;          // 8 or 16: each lane decodes 16 / DECODE_WARPS weight words per stage
  static constexpr int EPI_WARPS = 4;
  static constexpr int THREADS = (2 + DECODE_WARPS + EPI_WARPS) * 32;
  static constexpr int A_BYTES = 128 * KC * 2;           // 16 KiB
  static constexpr int B_BYTES = TT * KC * 2;            // 32 KiB
  static constexpr int Q_BYTES = 2 * 256 * 4;            // two slabs x 256 words
  static constexpr int M_BYTES = 2 * 128 * 4;
  static constexpr int S_BYTES = 256;                    // 128 halves
  static constexpr int A_OFF = 0;
  static constexpr int B_OFF = A_OFF + A_BYTES;
  static constexpr int Q_OFF = B_OFF + B_BYTES;
  static constexpr int M_OFF = Q_OFF + Q_BYTES;
  static constexpr int S_OFF = M_OFF + M_BYTES;
  static constexpr int STAGE_BYTES = (S_OFF + S_BYTES + 1023) / 1024 * 1024;
  static constexpr int ROWS_OFF = STAGES * STAGE_BYTES;                   // int [2][TT] output rows
  static constexpr int LUT_OFF = ROWS_OFF + 2 * TT * 4;
  static constexpr int PREFIX_OFF = LUT_OFF + 64;
  static constexpr int BAR_OFF = PREFIX_OFF + (kMaxSegments + 2) * 4;
  static constexpr int NUM_BARS = 3 * STAGES + 4;
  static constexpr int SMEM_BYTES = BAR_OFF + NUM_BARS * 8 + 16;
  static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = 512;
};

// PRMT selectors that place the two stored halves (v0 in bytes 0-1, v1 in bytes 2-3) of a 2:4 group
// at positions p0 = nib & 3 and p1 = nib >> 2 of four halves; low 16 bits build halves 0-1, high 16
// bits halves 2-3, selector 4 reads a zero byte.
__constant__ uint32_t kGroupSelector[16] = {0x44444410, 0x44441032, 0x44104432, 0x10444432, 0x44443210, 0x44441044,
                                            0x44103244, 0x10443244, 0x44324410, 0x44321044, 0x44104444, 0x10324444,
                                            0x32444410, 0x32441044, 0x32104444, 0x10444444};

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024
// bytes apart (stride byte offset), version 1 (sm_100), layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);        // start address
  d |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset
  d |= (uint64_t)1 << 46;                            // descriptor version
  d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: D fp32, A and B fp16, both K-major, N = 256, M = 128.
constexpr uint32_t kTcIdesc = (1u << 4) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kTcIdesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void sts64(uint32_t addr, uint32_t lo, uint32_t hi) {
  asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(lo), "r"(hi) : "memory");
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
  return v;
}

__global__ void __launch_bounds__(TcCfg::THREADS, 1)
delta_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_q,
                     const __grid_constant__ CUtensorMap tm_m, const __grid_constant__ CUtensorMap tm_s,
                     const GemmArgs a) {
  using Cfg = TcCfg;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int* rows_sm = reinterpret_cast<int*>(smem + Cfg::ROWS_OFF);
  uint32_t* lut_sm = reinterpret_cast<uint32_t*>(smem + Cfg::LUT_OFF);
  int* prefix = reinterpret_cast<int*>(smem + Cfg::PREFIX_OFF);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);   // TMA data of a stage landed
  uint64_t* aready_bar = full_bar + STAGES;                                // A tile of a stage written
  uint64_t* empty_bar = aready_bar + STAGES;                               // MMAs of a stage retired
  uint64_t* accready_bar = empty_bar + STAGES;                             // [2] accumulator complete
  uint64_t* accfree_bar = accready_bar + 2;                                // [2] accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfree_bar + 2);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  pdl_wait();   // launched with programmatic serialization: the predecessor's writes are visible after this
  int n_seg = a.n_seg_ptr ? *a.n_seg_ptr : a.n_seg;
  n_seg = max(0, min(n_seg, kMaxSegments));

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&aready_bar[s], Cfg::DECODE_WARPS);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&accready_bar[b], 1);
      mbar_init(&accfree_bar[b], Cfg::EPI_WARPS);
    }
    *dead = 0;
    fence_mbar_init();
  }
  if (tid < 16) lut_sm[tid] = kGroupSelector[tid];
  if (warp == 1) {
    // TMEM: all 512 columns (two 128 x 256 fp32 accumulators); this warp also frees them at the end.
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
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
  tc_fence_after();
  if (a.mode == kSegList) total_tiles = prefix[n_seg];
  else total_tiles = a.mode == kSegSingle ? (a.rows + Cfg::TT - 1) / Cfg::TT : a.rows;
  const uint32_t tmem_base = *tmem_slot;

  const int n_stripes = (a.N + 127) / 128;
  const int n_items = total_tiles * n_stripes;
  const int slabs = a.K / 32;
  const int k_chunks = a.K / Cfg::KC;
  const int groups = a.grouped ? a.K / 128 : 1;
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_x);
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_m);
      if (a.grouped) prefetch_tmap(&tm_s);
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      const uint32_t stage_tx = Cfg::B_BYTES + Cfg::Q_BYTES + Cfg::M_BYTES + (a.grouped ? Cfg::S_BYTES : 0);
      int st = 0;
      uint32_t phase = 0;
      for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, item);
        if (!w.ok) continue;
        for (int kc = 0; kc < k_chunks; ++kc) {
          mbar_wait(&empty_bar[st], phase ^ 1, dead);
          uint8_t* sbase = smem + st * Cfg::STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[st], stage_tx);
          tma_load_2d_hint(sbase + Cfg::B_OFF, &tm_x, kc * Cfg::KC, w.row0, &full_bar[st], pol_x);
          const int wrow = w.delta * slabs + kc * 2;
          tma_load_2d_hint(sbase + Cfg::Q_OFF, &tm_q, (w.col0 / 64) * 128, wrow, &full_bar[st], pol_w);
          tma_load_2d_hint(sbase + Cfg::M_OFF, &tm_m, (w.col0 / 64) * 64, wrow, &full_bar[st], pol_w);
          if (a.grouped)
            tma_load_2d_hint(sbase + Cfg::S_OFF, &tm_s, w.col0, w.delta * groups + kc / 2, &full_bar[st], pol_w);
          if (++st == STAGES) { st = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int st = 0;
      uint32_t phase = 0;
      uint32_t use[2] = {0, 0};
      int local = 0;
      for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, item);
        if (!w.ok) continue;
        const int buf = local & 1;
        mbar_wait(&accfree_bar[buf], (use[buf] & 1) ^ 1, dead);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * Cfg::TT;
        for (int kc = 0; kc < k_chunks; ++kc) {
          mbar_wait(&full_bar[st], phase, dead);
          mbar_wait(&aready_bar[st], phase, dead);
          tc_fence_after();
          const uint32_t sb = smem_base + st * Cfg::STAGE_BYTES;
          const uint64_t adesc = tc_smem_desc(sb + Cfg::A_OFF);
          const uint64_t bdesc = tc_smem_desc(sb + Cfg::B_OFF);
#pragma unroll
          for (int k = 0; k < Cfg::KC / 16; ++k)   // +32 bytes of K per instruction = +2 in the address field
            tc_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, (kc > 0 || k > 0) ? 1u : 0u);
          tc_commit(&empty_bar[st]);
          if (++st == STAGES) { st = 0; phase ^= 1; }
        }
        tc_commit(&accready_bar[buf]);
        ++use[buf];
        ++local;
      }
    }
  } else if (warp < 2 + Cfg::DECODE_WARPS) {
    // ------------------------------ decode warps: packed -> A tile ------------------------------
    // Warp dw handles column block cb and U row groups g of it; lane = (slab s, lane-in-quad m,
    // register j): it decodes weight word (s, cb, g, m, j) for each of its g.
    constexpr int U = 16 / Cfg::DECODE_WARPS;
    const int dw = warp - 2;
    const int cb = dw / (Cfg::DECODE_WARPS / 2);
    // Lane bits are (j high, s, m, j low): the 16 lanes of a half warp then hold two rows (j low) x eight
    // pieces, and when even-j lanes store their K-group-m piece while odd-j lanes store their
    // group-(m+4) piece (and the other way round in the next instruction) every 8-byte store of a half
    // warp lands in its own bank pair of the swizzled tile.
    const int s = (lane >> 3) & 1, m = (lane >> 1) & 3, j = ((lane >> 4) << 1) | (lane & 1);
    const bool jodd = lane & 1;
    uint32_t q_off[U], m_off[U], s_off[U], st_off[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = U * (dw % (Cfg::DECODE_WARPS / 2)) + u;
      q_off[u] = Cfg::Q_OFF + s * 1024 + cb * 512 + (4 * g + m) * 16 + j * 4;
      m_off[u] = Cfg::M_OFF + s * 512 + cb * 256 + (2 * (j & 1) + 32 * (j >> 1) + 4 * g) * 4;
      s_off[u] = Cfg::S_OFF + (cb * 64 + 8 * g + 2 * j) * 2;
      const int n0 = cb * 64 + 8 * g + j;            // block-0 row; block-1 row is n0 + 4
#pragma unroll
      for (int t = 0; t < 4; ++t) {                  // store t writes piece p: (n0, grp m), (n0, grp m+4), (n1, m), (n1, m+4)
        const int p = (t & 2) | ((t & 1) ^ (jodd ? 1 : 0));
        const int n = n0 + 4 * (p >> 1);
        const int kc8 = 8 * s + m + 4 * (p & 1);     // 8-byte piece index inside the 128-byte row
        st_off[u][t] = Cfg::A_OFF + (n >> 3) * 1024 + (n & 7) * 128 + ((((kc8 >> 1) ^ (n & 7))) << 4) + (kc8 & 1) * 8;
      }
    }
    const uint32_t lut_addr = smem_base + Cfg::LUT_OFF;
    int st = 0;
    uint32_t phase = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      const WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, item);
      if (!w.ok) continue;
      for (int kc = 0; kc < k_chunks; ++kc) {
        mbar_wait(&full_bar[st], phase, dead);
        const uint32_t sb = smem_base + st * Cfg::STAGE_BYTES;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t q = lds32(sb + q_off[u]);
          const uint2 mw = lds64(sb + m_off[u]);       // .x: K 0-15 of the slab, .y: K 16-31; low half n0, high half n1
          uint32_t v[4];                               // stored pairs of pieces 0..3
          int4x4_to_half2x2(q, v[0], v[1]);
          int4x4_to_half2x2(q >> 8, v[2], v[3]);
          if (a.grouped) {
            const uint32_t sc = lds32(sb + s_off[u]);  // (scale of n0, scale of n1)
            const uint32_t s0 = __byte_perm(sc, 0, 0x1010), s1 = __byte_perm(sc, 0, 0x3232);
            v[0] = hmul2_u32(v[0], s0); v[1] = hmul2_u32(v[1], s0);
            v[2] = hmul2_u32(v[2], s1); v[3] = hmul2_u32(v[3], s1);
          }
          const uint32_t nib[4] = {(mw.x >> (4 * m)) & 15u, (mw.y >> (4 * m)) & 15u, (mw.x >> (16 + 4 * m)) & 15u,
                                   (mw.y >> (16 + 4 * m)) & 15u};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int pa = t, pb = t ^ 1;              // odd-j lanes swap the two K groups of a row
            const uint32_t val = jodd ? v[pb] : v[pa];
            const uint32_t nb = jodd ? nib[pb] : nib[pa];
            // PRMT selector from the 16-entry table: byte q of sel picks the source bytes of output
            // half q (first stored value at position nb & 3, second at nb >> 2, zero elsewhere).
            const uint32_t sel = lds32(lut_addr + nb * 4);
            sts64(sb + st_off[u][t], __byte_perm(val, 0, sel), __byte_perm(val, 0, sel >> 16));
          }
        }
        fence_proxy_async();      // the tensor core reads the tile through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&aready_bar[st]);
        if (++st == STAGES) { st = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int ew = warp - 2 - Cfg::DECODE_WARPS;
    const int quad = warp & 3;                        // TMEM lanes this warp may touch: 32*quad .. +31
    uint32_t use[2] = {0, 0};
    int local = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      const WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, item);
      if (!w.ok) continue;
      const int buf = local & 1;
      int* rows = rows_sm + buf * Cfg::TT;
      // Output rows of the tile's tokens (each epilogue warp fills a quarter; barrier 4 = these warps).
      for (int t = ew * 32 + lane; t < Cfg::TT; t += Cfg::EPI_WARPS * 32) {
        int r = -1;
        if (t < w.valid) {
          r = w.row0 + t;
          if (a.row_map) r = a.row_map[r];
          if (r < 0 || r >= a.rows) r = -1;
        }
        rows[t] = r;
      }
      const int n = w.col0 + quad * 32 + lane;        // this thread's output feature
      float sf = 1.f;
      if (!a.grouped && n < a.N) sf = __half2float(a.scales[(size_t)w.delta * a.N + n]);
      named_bar_sync(4, Cfg::EPI_WARPS * 32);
      mbar_wait(&accready_bar[buf], use[buf] & 1, dead);
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * Cfg::TT;
      const int nbatch = (w.valid + 31) >> 5;
      for (int b = 0; b < nbatch; ++b) {
        uint32_t v[32];
        tc_ld32(taddr + b * 32, v);
        tc_wait_ld();
        if (n < a.N) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int r = rows[b * 32 + c];
            if (r >= 0) {
              __half* yp = a.y + (size_t)r * a.N + n;
              float val = __uint_as_float(v[c]) * sf;
              if (a.accumulate) val += __half2float(*yp);
              *yp = __float2half_rn(val);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&accfree_bar[buf]);
      named_bar_sync(4, Cfg::EPI_WARPS * 32);          // rows[] of this buffer may be rewritten two items later
      ++use[buf];
      ++local;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
  }
}

}  // namespace trb
