// Grouped 2:4-sparse int4 delta GEMM for decode-sized token tiles (HBM-bound regime).
//
// One persistent launch serves every (token segment, 64*SW-column stripe) work item of a batch:
// a producer warp streams packed weights, 2:4 metadata, scales and the activation tile into a
// ring of shared-memory stages with TMA (cp.async.bulk.tensor + mbarrier transaction counts),
// eight consumer warps turn nibbles into fp16 in registers and issue 2:4-sparse tensor-core
// MMAs with the weights as the sparse operand (output features on the MMA M dimension, tokens
// on N).  Every delta is read from HBM once per token tile; no split-K across CTAs, no locks.
//
// The work done per (32-K slab, 64-column block) follows the packed format's own fragment
// order (reference: triteia/python/ops/utils/sparsity.py:35-61 for the nibble order,
// :134-161 for the metadata order; the consuming kernel in the reference is
// triteia/csrc/ops/marlin.cuh:337-387): lane i owns words 4i..4i+3 of the block's 128 weight
// words and metadata words i and 32+i of its 64 metadata words.
#pragma once

#include "common.cuh"

namespace trb {

constexpr int kMaxSegments = 1024;

// kSegList: segments of any length (tiles counted per segment through a prefix table in shared memory,
// at most kMaxSegments segments per launch); kSegSingle: one segment = all rows, delta 0;
// kSegIdentity: row r is its own segment with delta r; kSegTiles: the lists hold ready-made tiles
// (at most Cfg::TT rows each, as the router writes them), no limit on their number.
enum SegMode { kSegList = 0, kSegSingle = 1, kSegIdentity = 2, kSegTiles = 3 };

struct GemmArgs {
  const int* seg_delta;   // [n_seg] delta id per segment (kSegList)
  const int* seg_start;   // [n_seg] first row of the segment in x / y
  const int* seg_count;   // [n_seg] rows in the segment
  const int* n_seg_ptr;   // device scalar with the segment count, or nullptr -> n_seg
  int n_seg;
  int mode;
  int rows;               // rows of x and y
  int N, K;
  int num_deltas;
  int grouped;            // 0: scales [D,1,N] applied in the epilogue; 1: [D,K/128,N]
  const __half* scales;
  __half* y;
  const int* row_map;     // nullptr, or output row of each x row (scatter through the router's perm)
  int accumulate;         // y += result instead of y = result
  // Sharded path, results stored straight into the token owners' output over NVLink: x row
  // r * chunk_rows + q came from rank r, whose token row is entry chunk_rows + q of the int32 id row
  // that closes chunk r of the exchange buffer `xchg` (rows of xchg_row_bytes); the result goes to
  // that row of y_peers[r] (nullptr: plain y).
  __half* const* y_peers;
  const unsigned char* xchg;
  long long xchg_row_bytes;
  int chunk_rows;
  // Tail K split (8-token tiles): when the last round of work items covers at most half of the
  // CTAs, each of its items is cut along K into `parts` pieces taken by neighbouring CTAs.  Every
  // piece writes its fp32 partial tile to `ksplit_buf` (kKsplitSlots slots of kKsplitSlotFloats),
  // bumps the item's counter in `ksplit_cnt` (kKsplitItems ints, zero on entry, zero again on
  // exit) and leaves; the piece that arrives last adds all pieces in a fixed order and runs the
  // epilogue.  Nobody waits for anybody.  nullptr: no split.
  float* ksplit_buf;
  int* ksplit_cnt;
};
constexpr int kKsplitItems = 74;              // at most half a grid of tail items is split
constexpr int kKsplitSlots = 148;             // pieces over all tail items
constexpr int kKsplitSlotFloats = 256 * 8;    // one 8-token x 256-column fp32 tile
constexpr size_t kKsplitBufBytes = (size_t)kKsplitSlots * kKsplitSlotFloats * 4;

template <int NB_, int SW_, int KQ_, int KS_, int STAGES_>
struct GemmCfg {
  static constexpr int NB = NB_;          // token blocks of 8 per tile
  static constexpr int SW = SW_;          // 64-column blocks per stripe
  static constexpr int KQ = KQ_;          // warps sharing one column block (split over slabs)
  static constexpr int KS = KS_;          // 32-K slabs per pipeline stage
  static constexpr int STAGES = STAGES_;
  static constexpr int CW = SW * KQ;                // consumer warps
  static constexpr int CTHREADS = CW * 32;
  static constexpr int THREADS = CTHREADS + 32;     // + one producer warp
  static_assert(CW == 8, "8 consumer warps");
  static_assert(NB == 1 || NB == 2 || NB == 4, "tile classes are 1, 2 and 4 token blocks");
  static_assert(KQ == 1 || KQ == 2 || KQ == 4, "the K split must divide the four j's of a fragment");
  static_assert(KS % 4 == 0 && KS % KQ == 0 && KS % 2 == 0, "stage must hold whole scale groups");
  static_assert((KS / KQ) <= 4 && 4 % (KS / KQ) == 0 && KS <= 32, "a warp's slabs of a stage share one scale group");
  static constexpr int TT = NB * 8;                 // tokens per tile
  static constexpr int QB = SW >= 2 ? 2 : 1;        // column blocks per weight TMA box
  static constexpr int NQBOX = SW / QB;
  static constexpr int NXBOX = KS / 2;              // 64-half boxes of activations per stage
  static constexpr int X_BOX_BYTES = TT * 128;
  static constexpr int X_BYTES = NXBOX * X_BOX_BYTES;
  static constexpr int Q_BYTES = KS * SW * 512;
  static constexpr int M_BYTES = KS * SW * 256;
  static constexpr int SB = SW >= 4 ? 4 : SW;       // column blocks per scale TMA box (a box dimension is at most 256)
  static constexpr int NSBOX = SW / SB;
  static constexpr int S_BOX_BYTES = (KS / 4) * SB * 128;
  static constexpr int S_BYTES = NSBOX * S_BOX_BYTES;
  static constexpr int X_OFF = 0;
  static constexpr int Q_OFF = (X_BYTES + 1023) / 1024 * 1024;
  static constexpr int M_OFF = Q_OFF + Q_BYTES;
  static constexpr int S_OFF = M_OFF + M_BYTES;
  static constexpr int STAGE_BYTES = (S_OFF + S_BYTES + 1023) / 1024 * 1024;
  static constexpr int RED_BUFS = KQ - 1;                     // partner-warp reduction buffers
  static constexpr int NBH = NB < 2 ? NB : 2;                 // token blocks exchanged per round
  static constexpr int RED_BUF_FLOATS = 16 * NBH * SW * 32;
  static constexpr int RED_FLOATS = RED_BUFS * RED_BUF_FLOATS;
  static constexpr int RED_OFF = STAGES * STAGE_BYTES;
  static constexpr int PREFIX_OFF = RED_OFF + RED_FLOATS * 4;
  static constexpr int BAR_OFF = PREFIX_OFF + (kMaxSegments + 2) * 4;
  // Staging of result tiles that leave for other GPUs: per column block 8 tokens x 64 halves, then
  // the 8 tokens' destination rows.
  static constexpr int STG_OFF = (BAR_OFF + 2 * STAGES * 8 + 16 + 15) / 16 * 16;
  static constexpr int STG_BLOCK_BYTES = 8 * 64 * 2 + 32;
  static constexpr int SMEM_BYTES = STG_OFF + SW * STG_BLOCK_BYTES;
  static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;  // slack to align the base to 1 KiB
};

struct WorkItem {
  int delta, row0, valid, col0;
  bool ok;
};

// The u-th unit of work of CTA b: a whole item in the full rounds, a K range of an item in the tail.
struct WorkUnit {
  int item, ks0, ks1, part, parts, tail;
};
struct TailSplit {
  int r_full, r_tail, parts, units;   // units = this CTA's number of work units
};
__device__ __forceinline__ TailSplit tail_split(int n_items, int k_stages, int grid, int b, bool allowed) {
  TailSplit t;
  t.r_full = n_items / grid;
  t.r_tail = n_items - t.r_full * grid;
  t.parts = 1;
  if (allowed && t.r_tail > 0 && 2 * t.r_tail <= grid && t.r_tail <= kKsplitItems) {
    int s = grid / t.r_tail;
    s = s > 8 ? 8 : s;
    s = s > k_stages ? k_stages : s;
    int p = 1;
    while (2 * p <= s) p *= 2;
    while (p > 1 && (k_stages % p != 0 || t.r_tail * p > kKsplitSlots)) p >>= 1;   // equal K ranges, slots for all
    t.parts = p;
  }
  t.units = t.r_full + (b < t.r_tail * t.parts ? 1 : 0);
  return t;
}
__device__ __forceinline__ WorkUnit work_unit(const TailSplit& t, int u, int grid, int b, int k_stages) {
  WorkUnit w;
  if (u < t.r_full) {
    w.item = b + u * grid; w.ks0 = 0; w.ks1 = k_stages; w.part = 0; w.parts = 1; w.tail = 0;
  } else {
    w.tail = b / t.parts;
    w.item = t.r_full * grid + w.tail;
    w.part = b - w.tail * t.parts;
    w.parts = t.parts;
    const int len = k_stages / t.parts;
    w.ks0 = w.part * len;
    w.ks1 = w.ks0 + len;
  }
  return w;
}

// Tile t of the batch -> (segment, tile inside the segment); item = tile * n_stripes + stripe.
template <class Cfg>
__device__ __forceinline__ WorkItem decode_item(const GemmArgs& a, const int* prefix, int n_seg,
                                                int n_stripes, int item) {
  WorkItem w;
  const int tile = item / n_stripes;
  const int stripe = item - tile * n_stripes;
  int seg, tin;
  if (a.mode == kSegSingle) {
    seg = 0;
    tin = tile;
  } else if (a.mode == kSegIdentity || a.mode == kSegTiles) {
    seg = tile;
    tin = 0;
  } else {
    int lo = 0, hi = n_seg;  // largest seg with prefix[seg] <= tile
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid] <= tile) lo = mid; else hi = mid;
    }
    seg = lo;
    tin = tile - prefix[seg];
  }
  int delta, start, count;
  if (a.mode == kSegSingle) {
    delta = 0; start = 0; count = a.rows;
  } else if (a.mode == kSegIdentity) {
    delta = seg; start = seg; count = 1;
  } else {
    delta = a.seg_delta[seg]; start = a.seg_start[seg]; count = a.seg_count[seg];
  }
  w.delta = delta;
  w.row0 = start + tin * Cfg::TT;
  w.valid = min(Cfg::TT, count - tin * Cfg::TT);
  w.col0 = stripe * Cfg::SW * 64;
  // Never trust a list entry with the address arithmetic: bad entries are skipped.
  w.ok = delta >= 0 && delta < a.num_deltas && start >= 0 && count >= 0 &&
         start + count <= a.rows && w.valid > 0;
  return w;
}

// Where a consumer warp stands in the stage ring, carried from one work unit to the next.
struct PipeState {
  int st;
  uint32_t phase;
  bool first_item;
};

// One work unit of a consumer warp: a tile of NB token blocks against one stripe (or a K range of it).
template <class Cfg, int NB>
__device__ __forceinline__ PipeState run_unit_body(const GemmArgs& a, uint8_t* smem, PipeState ps, const WorkUnit wu,
                                                   const WorkItem w) {
  constexpr int SW = Cfg::SW, KQ = Cfg::KQ, KS = Cfg::KS, STAGES = Cfg::STAGES;
  float* red = reinterpret_cast<float*>(smem + Cfg::RED_OFF);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  volatile int* dead = reinterpret_cast<volatile int*>(empty_bar + STAGES);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slabs = a.K / 32;
  const int cb = warp / KQ;   // column block of the stripe
  const int kq = warp % KQ;   // which share of each stage's slabs
  const int g8 = lane >> 2;   // quad index: MMA row group / token inside a block of 8
  const int m4 = lane & 3;
  constexpr int SPW = KS / KQ;  // slabs per warp per stage
  const int box = cb / Cfg::QB, within = cb % Cfg::QB;
  // Per-lane byte offsets inside a stage.
  const uint32_t q_off = Cfg::Q_OFF + box * (KS * Cfg::QB * 512) + within * 512 + lane * 16 + kq * SPW * (Cfg::QB * 512);
  const uint32_t m_off = Cfg::M_OFF + box * (KS * Cfg::QB * 256) + within * 256 + lane * 4 + kq * SPW * (Cfg::QB * 256);
  const uint32_t s_off = Cfg::S_OFF + (cb / Cfg::SB) * Cfg::S_BOX_BYTES + ((kq * SPW) / 4) * (Cfg::SB * 128) +
                         (cb % Cfg::SB) * 128 + g8 * 16;
  const uint32_t smem_base = smem_u32(smem);
  int st = ps.st;
  uint32_t phase = ps.phase;
  bool first_item = ps.first_item;
  constexpr int JW = 4 / KQ;   // accumulator column pairs (j) that each partner warp finishes
  // A warp's slabs of one stage lie inside one scale group, so their integer-level products are
  // accumulated on their own and scaled once per stage in fp32 (small token tiles); large token
  // tiles scale every weight in fp16 instead, which costs less than scaling many accumulators.
  constexpr bool kPostScale = (NB <= 2);
  constexpr bool kBulkLoad = (NB == 1);   // larger tiles would spill: they load slab by slab
  constexpr uint32_t XBOX = NB * 1024;    // bytes of one 64-K activation box of this class
  // ldmatrix row address of slab i of this warp: 16-byte chunk 4*slab + lane/8 of the stage's K
  // range lives in activation box chunk/8 at swizzled chunk position (chunk%8) ^ (row%8).
  uint32_t x_off[SPW];
#pragma unroll
  for (int i = 0; i < SPW; ++i) {
    const int chunk = (kq * SPW + i) * 4 + (lane >> 3);
    x_off[i] = Cfg::X_OFF + (chunk >> 3) * XBOX + (lane & 7) * 128 + ((((chunk & 7) ^ (lane & 7))) << 4);
  }
  const int nbv = (w.valid + 7) >> 3;
  const bool col_ok = w.col0 + cb * 64 < a.N;

  // Epilogue operands fetched now, used after the K loop: output rows of this lane's tokens and
  // (per-channel mode) the scales of the two columns of each j this warp finishes.
  const int colb = w.col0 + cb * 64 + g8 * 8;
  int orow[NB][2];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int t = nb * 8 + 2 * m4 + h;
      int r = -1;
      if (t < w.valid) {
        r = w.row0 + t;
        if (a.row_map) r = a.row_map[r];
        if (r < 0 || r >= a.rows) r = -1;
        if (a.y_peers && r >= 0) {
          // (source rank << 20) | token row on that rank
          const int pr = r / a.chunk_rows, pq = r - pr * a.chunk_rows;
          const int* ids = reinterpret_cast<const int*>(a.xchg + ((long long)pr * a.chunk_rows + a.chunk_rows - 1) * a.xchg_row_bytes);
          const int trow = ids[a.chunk_rows + pq];
          r = (trow >= 0 && trow < a.chunk_rows - 1) ? ((pr << 20) | trow) : -1;   // a peer's output has chunk_rows - 1 rows
        }
      }
      orow[nb][h] = r;
    }
  float sfa[JW], sfb[JW];
#pragma unroll
  for (int jj = 0; jj < JW; ++jj) {
    sfa[jj] = 1.f;
    sfb[jj] = 1.f;
    if (!a.grouped && col_ok) {
      const __half* sp = a.scales + (size_t)w.delta * a.N + colb + kq * JW + jj;
      sfa[jj] = __half2float(sp[0]);
      sfb[jj] = __half2float(sp[4]);
    }
  }

  float acc[4][NB][4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[j][nb][c] = 0.f;

  for (int ks = wu.ks0; ks < wu.ks1; ++ks) {
    mbar_wait(&full_bar[st], phase, dead);
    const uint32_t sb = smem_base + st * Cfg::STAGE_BYTES;

    // One stage of this warp's slabs.  FULL: every slab of the stage exists (no per-slab test, so
    // the four slabs form one straight-line block the compiler can interleave).  GROUPED selects
    // the scale handling at compile time.
    auto run_stage = [&](auto full_tag, auto grouped_tag) {
      constexpr bool FULL = decltype(full_tag)::value;
      constexpr bool GROUPED = decltype(grouped_tag)::value;
      constexpr bool POST = kPostScale && GROUPED;
      uint32_t scs[4] = {0, 0, 0, 0};
      if constexpr (GROUPED) {
        const uint4 sc = lds128(sb + s_off);
        scs[0] = sc.x; scs[1] = sc.y; scs[2] = sc.z; scs[3] = sc.w;
      }
      float accg[4][NB][4];   // integer-level partial sums of this warp's slabs (POST)

      // MMAs of one slab from registers: q4 = the lane's four weight words, e0/e1 = its two
      // metadata words, bf = activation fragments per token block.
      auto compute_slab = [&](int i, const uint4& q4, uint32_t e0, uint32_t e1, const uint32_t (&bf)[NB][4]) {
        const uint32_t qs[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t lo0, hi0, lo1, hi1;
          int4x4_to_half2x2(qs[j], lo0, hi0);
          int4x4_to_half2x2(qs[j] >> 8, lo1, hi1);
          if constexpr (GROUPED && !kPostScale) {
            const uint32_t s0 = __byte_perm(scs[j], 0, 0x1010);  // scale of column j, both halves
            const uint32_t s1 = __byte_perm(scs[j], 0, 0x3232);  // scale of column j + 4
            lo0 = hmul2_u32(lo0, s0); hi0 = hmul2_u32(hi0, s0);
            lo1 = hmul2_u32(lo1, s1); hi1 = hmul2_u32(hi1, s1);
          }
          const uint32_t e = (j < 2) ? e0 : e1;
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            if (NB == 1 || nb < nbv) {
              if constexpr (POST) {
                if (i == 0) {
                  if (j & 1) mma_sp_m16n8k32_zero<1>(accg[j][nb], lo0, lo1, hi0, hi1, bf[nb], e);
                  else       mma_sp_m16n8k32_zero<0>(accg[j][nb], lo0, lo1, hi0, hi1, bf[nb], e);
                } else {
                  if (j & 1) mma_sp_m16n8k32<1>(accg[j][nb], lo0, lo1, hi0, hi1, bf[nb], e);
                  else       mma_sp_m16n8k32<0>(accg[j][nb], lo0, lo1, hi0, hi1, bf[nb], e);
                }
              } else {
                if (j & 1) mma_sp_m16n8k32<1>(acc[j][nb], lo0, lo1, hi0, hi1, bf[nb], e);
                else       mma_sp_m16n8k32<0>(acc[j][nb], lo0, lo1, hi0, hi1, bf[nb], e);
              }
            }
          }
        }
      };

      if constexpr (kBulkLoad) {
        // Small token tiles: one slab at a time into registers (the warp's whole share of the stage at
        // once needs 40 registers more and spilled inside this loop: 85 -> 81 us on the decode
        // benchmark), the stage handed back to the producer right after the last slab's loads (the
        // arrive is a release: the loads above are performed before it is observed), before its math.
#pragma unroll
        for (int i = 0; i < SPW; ++i) {
          uint4 q4 = make_uint4(0u, 0u, 0u, 0u);
          uint32_t e0 = 0u, e1 = 0u, bf[NB][4];
          const bool have = FULL || ks * KS + kq * SPW + i < slabs;
          if (have) {
            q4 = lds128(sb + q_off + i * (Cfg::QB * 512));
            e0 = lds32(sb + m_off + i * (Cfg::QB * 256));
            e1 = lds32(sb + m_off + i * (Cfg::QB * 256) + 128);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
              if (NB == 1 || nb < nbv) ldmatrix_x4(bf[nb], sb + x_off[i] + nb * 1024);
          }
          if (i == SPW - 1) {   // the warp's last loads of the stage are out: hand the stage back
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[st]);
          }
          if (have) compute_slab(i, q4, e0, e1, bf);
        }
      } else {
        // 32-token tiles keep 64 accumulators per lane: their slabs run one after the other.
        constexpr int kSlabUnroll = NB >= 4 ? 1 : SPW;
#pragma unroll kSlabUnroll
        for (int i = 0; i < SPW; ++i) {
          if (FULL || ks * KS + kq * SPW + i < slabs) {
            const uint4 q4 = lds128(sb + q_off + i * (Cfg::QB * 512));
            const uint32_t e0 = lds32(sb + m_off + i * (Cfg::QB * 256));
            const uint32_t e1 = lds32(sb + m_off + i * (Cfg::QB * 256) + 128);
            uint32_t bf[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
              if (NB == 1 || nb < nbv) ldmatrix_x4(bf[nb], sb + x_off[i] + nb * 1024);
            compute_slab(i, q4, e0, e1, bf);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[st]);
      }
      // A scale group is whole or absent (K is a multiple of 128): slab 0 of the warp decides.
      if (POST && (FULL || ks * KS + kq * SPW < slabs)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&scs[j]));
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            if (NB == 1 || nb < nbv) {
              acc[j][nb][0] = fmaf(accg[j][nb][0], sf.x, acc[j][nb][0]);
              acc[j][nb][1] = fmaf(accg[j][nb][1], sf.x, acc[j][nb][1]);
              acc[j][nb][2] = fmaf(accg[j][nb][2], sf.y, acc[j][nb][2]);
              acc[j][nb][3] = fmaf(accg[j][nb][3], sf.y, acc[j][nb][3]);
            }
          }
        }
      }
    };
    if (col_ok) {
      const bool full = (ks + 1) * KS <= slabs;
      if (a.grouped) {
        if (full) run_stage(std::true_type{}, std::true_type{});
        else run_stage(std::false_type{}, std::true_type{});
      } else {
        if (full) run_stage(std::true_type{}, std::false_type{});
        else run_stage(std::false_type{}, std::false_type{});
      }
    } else {
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[st]);
    }
    if (++st == STAGES) { st = 0; phase ^= 1; }
  }

  // Partner warps (same column block) own identical fragments.  Each of them finishes the j's
  // [kq*JW, (kq+1)*JW): it hands its partial sums of the other j's to their owners through shared
  // memory, adds the partners' partials to its own in a fixed order, and writes its columns.
  // The exchange runs in rounds of at most two token blocks (the buffer holds that much).
  // Only the KQ warps of a column block meet (two hardware barriers per column block): the one
  // before the stores keeps a round's partials until every reader of the previous round is done,
  // the other separates stores from loads.
  if constexpr (KQ > 1) {
    constexpr int CT = Cfg::CTHREADS;
    constexpr int LANES = SW * 32;
    constexpr int NBH = NB < 2 ? NB : 2;
#pragma unroll
    for (int h0 = 0; h0 < NB; h0 += NBH) {
      if (!first_item) named_bar_sync(6 + 2 * cb, KQ * 32);
      first_item = false;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int owner = j / JW;
        if (owner != kq) {
          const int slot = kq < owner ? kq : kq - 1;
          float* dst = red + (((owner * (KQ - 1) + slot) * JW + (j % JW)) * NBH * 4) * LANES + cb * 32 + lane;
#pragma unroll
          for (int nb = 0; nb < NBH; ++nb)
#pragma unroll
            for (int c = 0; c < 4; ++c) dst[(nb * 4 + c) * LANES] = acc[j][h0 + nb][c];
        }
      }
      named_bar_sync(7 + 2 * cb, KQ * 32);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j / JW == kq) {
#pragma unroll
          for (int slot = 0; slot < KQ - 1; ++slot) {
            const float* src = red + (((kq * (KQ - 1) + slot) * JW + (j % JW)) * NBH * 4) * LANES + cb * 32 + lane;
#pragma unroll
            for (int nb = 0; nb < NBH; ++nb)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[j][h0 + nb][c] += src[(nb * 4 + c) * LANES];
          }
        }
      }
    }
  }

  // A piece of a K-split item: park the fp32 partial tile, count in; all but the last arriver are
  // done with the item.  The last arriver replaces its registers with the sum of every piece's
  // tile in piece order (its own included), so the result does not depend on who came last.
  if constexpr (NB == 1) {
    if (wu.parts > 1) {
      // slot of piece p of tail item t: ((t * parts + p) * 2 + jj) * CT float4s, this thread's at + tid
      float4* tile = reinterpret_cast<float4*>(a.ksplit_buf) + (size_t)(wu.tail * wu.parts) * (kKsplitSlotFloats / 4) +
                     (warp * 32 + lane);
      // (static accumulator indices under a predicate, as in the epilogue: a run-time index would
      // push the accumulators out of registers)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (j / JW == kq)
          __stcg(tile + (wu.part * 2 + j % JW) * Cfg::CTHREADS,
                 make_float4(acc[j][0][0], acc[j][0][1], acc[j][0][2], acc[j][0][3]));
      // One acq_rel atomic by one thread between two CTA barriers orders every thread's tile
      // stores before the count (release, cumulative over the barrier) and every thread's tile
      // loads after it (acquire).  A tail piece is a CTA's last unit: the flag word is used once.
      named_bar_sync(3, Cfg::CTHREADS);
      volatile int* flag = dead + 1;
      if (warp == 0 && lane == 0) {
        int old;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(a.ksplit_cnt + wu.tail) : "memory");
        *flag = old;
      }
      named_bar_sync(3, Cfg::CTHREADS);
      if (*flag != wu.parts - 1) return PipeState{st, phase, first_item};
      if (warp == 0 && lane == 0) a.ksplit_cnt[wu.tail] = 0;   // back to zero for the next launch
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j / JW == kq) {
          float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
          for (int p = 0; p < wu.parts; ++p) {
            const float4 v = __ldcg(tile + (p * 2 + j % JW) * Cfg::CTHREADS);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
          }
          acc[j][0][0] = sum.x; acc[j][0][1] = sum.y; acc[j][0][2] = sum.z; acc[j][0][3] = sum.w;
        }
      }
    }
  }
  if constexpr (NB == 1 && KQ > 1) {
    if (a.y_peers != nullptr) {
      // Results that leave for other GPUs go out in 16-byte pieces: the partner warps of a column
      // block put their 8-token x 64-column tile together in shared memory, meet once on their own
      // barrier, and each lane stores eight consecutive features of one token over NVLink, instead
      // of eight 2-byte stores per lane.  Nothing here is CTA-wide.  The tile is written again only
      // after the next unit's exchange barriers, which a partner reaches after its loads below.
      __half* tile = reinterpret_cast<__half*>(smem + Cfg::STG_OFF + cb * Cfg::STG_BLOCK_BYTES);
      int* trow = reinterpret_cast<int*>(tile + 8 * 64);
      if (col_ok) {
        __half* tp = tile + g8 * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j / JW == kq) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              tp[(2 * m4 + h) * 64 + j] = __float2half_rn(acc[j][0][h] * sfa[j % JW]);
              tp[(2 * m4 + h) * 64 + j + 4] = __float2half_rn(acc[j][0][2 + h] * sfb[j % JW]);
            }
          }
        }
      }
      if (kq == 0 && g8 == 0) {
        trow[2 * m4] = orow[0][0];
        trow[2 * m4 + 1] = orow[0][1];
      }
      named_bar_sync(7 + 2 * cb, KQ * 32);
      for (int p = kq * 32 + lane; p < 64; p += KQ * 32) {       // 8 tokens x 8 pieces
        const int t = p >> 3, c = (p & 7) * 8;
        const int r = trow[t];
        if (r >= 0 && col_ok) {
          uint4 o = *reinterpret_cast<const uint4*>(tile + t * 64 + c);
          uint4* yp = reinterpret_cast<uint4*>(a.y_peers[r >> 20] + (size_t)(r & ((1 << 20) - 1)) * a.N + w.col0 + cb * 64 + c);
          if (a.accumulate) {
            const uint4 old = *yp;
            __half2* oh = reinterpret_cast<__half2*>(&o);
            const __half2* ph = reinterpret_cast<const __half2*>(&old);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x2 = __half22float2(oh[e]), y2 = __half22float2(ph[e]);
              oh[e] = __floats2half2_rn(x2.x + y2.x, x2.y + y2.y);
            }
          }
          *yp = o;
        }
      }
      return PipeState{st, phase, first_item};
    }
  }
  if (col_ok) {
    // acc[j][nb][h] is (column colb + j, token nb*8 + 2*m4 + h); acc[j][nb][2 + h] is column colb + 4 + j.
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j / JW == kq) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int r = orow[nb][h];
            if (r >= 0 && (NB == 1 || nb < nbv)) {
              __half* yp;
              if (a.y_peers) {
                yp = a.y_peers[r >> 20] + (size_t)(r & ((1 << 20) - 1)) * a.N + colb + j;
              } else {
                yp = a.y + (size_t)r * a.N + colb + j;
              }
              float va = acc[j][nb][h] * sfa[j % JW];
              float vb = acc[j][nb][2 + h] * sfb[j % JW];
              if (a.accumulate) {
                va += __half2float(yp[0]);
                vb += __half2float(yp[4]);
              }
              yp[0] = __float2half_rn(va);
              yp[4] = __float2half_rn(vb);
            }
          }
        }
      }
    }
  }
  return PipeState{st, phase, first_item};
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
delta_gemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_q,
                  const __grid_constant__ CUtensorMap tm_m, const __grid_constant__ CUtensorMap tm_s,
                  const __grid_constant__ GemmArgs a) {
  constexpr int NBMAX = Cfg::NB, SW = Cfg::SW, KS = Cfg::KS, STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* red = reinterpret_cast<float*>(smem + Cfg::RED_OFF);
  int* prefix = reinterpret_cast<int*>(smem + Cfg::PREFIX_OFF);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  volatile int* dead = reinterpret_cast<volatile int*>(empty_bar + STAGES);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  pdl_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], Cfg::CW);
    }
    *dead = 0;
    fence_mbar_init();
  }
  pdl_wait();   // everything below reads what the kernels launched before this one wrote
  if (a.mode == kSegTiles && a.n_seg_ptr != nullptr && *a.n_seg_ptr <= 0) return;   // the router left this list empty

  int n_seg = a.n_seg_ptr ? *a.n_seg_ptr : a.n_seg;
  n_seg = max(0, min(n_seg, a.mode == kSegTiles ? a.n_seg : kMaxSegments));

  // Tiles-per-segment prefix sums (list mode).  Warp 0 scans 32 segments per step.
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
    __syncthreads();
    total_tiles = prefix[n_seg];
  } else {
    __syncthreads();
    total_tiles = a.mode == kSegTiles ? n_seg : (a.mode == kSegSingle ? (a.rows + Cfg::TT - 1) / Cfg::TT : a.rows);
  }

  const int n_stripes = (a.N + SW * 64 - 1) / (SW * 64);
  const int n_items = total_tiles * n_stripes;
  const int slabs = a.K / 32;
  const int k_stages = (slabs + KS - 1) / KS;
  const int groups = a.grouped ? a.K / 128 : 1;
  // Work units of this CTA: whole items in the full rounds, then (maybe) a K range of a tail item.
  const TailSplit split = tail_split(n_items, k_stages, (int)gridDim.x, (int)blockIdx.x,
                                     NBMAX == 1 && SW * 512 <= kKsplitSlotFloats && a.ksplit_buf != nullptr);

  if (warp == Cfg::CW) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_x);
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_m);
      if (a.grouped) prefetch_tmap(&tm_s);
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      const uint32_t stage_tx = Cfg::X_BYTES + Cfg::Q_BYTES + Cfg::M_BYTES + (a.grouped ? Cfg::S_BYTES : 0);
      int st = 0;
      uint32_t phase = 0;
      for (int u = 0; u < split.units; ++u) {
        const WorkUnit wu = work_unit(split, u, (int)gridDim.x, (int)blockIdx.x, k_stages);
        const WorkItem w = decode_item<Cfg>(a, prefix, n_seg, n_stripes, wu.item);
        if (!w.ok) continue;
        for (int ks = wu.ks0; ks < wu.ks1; ++ks) {
          mbar_wait(&empty_bar[st], phase ^ 1, dead);
          uint8_t* sbase = smem + st * Cfg::STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[st], stage_tx);
#pragma unroll
          for (int b = 0; b < Cfg::NXBOX; ++b)
            tma_load_2d_hint(sbase + Cfg::X_OFF + b * Cfg::X_BOX_BYTES, &tm_x, ks * KS * 32 + b * 64, w.row0,
                             &full_bar[st], pol_x);
          const int wrow = w.delta * slabs + ks * KS;
#pragma unroll
          for (int b = 0; b < Cfg::NQBOX; ++b) {
            tma_load_2d_hint(sbase + Cfg::Q_OFF + b * (KS * Cfg::QB * 512), &tm_q,
                             (w.col0 / 64 + b * Cfg::QB) * 128, wrow, &full_bar[st], pol_w);
            tma_load_2d_hint(sbase + Cfg::M_OFF + b * (KS * Cfg::QB * 256), &tm_m,
                             (w.col0 / 64 + b * Cfg::QB) * 64, wrow, &full_bar[st], pol_w);
          }
          if (a.grouped) {
#pragma unroll
            for (int b = 0; b < Cfg::NSBOX; ++b)
              tma_load_2d_hint(sbase + Cfg::S_OFF + b * Cfg::S_BOX_BYTES, &tm_s, w.col0 + b * Cfg::SB * 64,
                               w.delta * groups + ks * (KS / 4), &full_bar[st], pol_w);
          }
          if (++st == STAGES) { st = 0; phase ^= 1; }
        }
      }
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  PipeState ps{0, 0u, true};
  WorkItem w_next{};

  if (split.units > 0)
    w_next = decode_item<Cfg>(a, prefix, n_seg, n_stripes,
                              work_unit(split, 0, (int)gridDim.x, (int)blockIdx.x, k_stages).item);
  for (int u = 0; u < split.units; ++u) {
    const WorkUnit wu = work_unit(split, u, (int)gridDim.x, (int)blockIdx.x, k_stages);
    const WorkItem w = w_next;
    // Descriptor of the next item: its global loads are in flight during this item's K loop.
    if (u + 1 < split.units)
      w_next = decode_item<Cfg>(a, prefix, n_seg, n_stripes,
                                work_unit(split, u + 1, (int)gridDim.x, (int)blockIdx.x, k_stages).item);
    if (!w.ok) continue;
    ps = run_unit_body<Cfg, NBMAX>(a, smem, ps, wu, w);
  }
}

}  // namespace trb
