// On-GPU packer: fp16 weight [K, N] + logical scales [G, N] -> the packed int4 + 2:4 format
// (qweight int32 [K/32, 2N], meta int16 [N, K/16] in its physical order, stored scales fp16 [G, N]).
// The producer side of the format, as a kernel: the reference packs on the host with numpy in a
// Python loop (triteia/python/nn/linear.py:79-141 on top of the compressor and metadata reorder of
// triteia/python/ops/utils/sparsity.py:134-161, 167-290).
//
// One thread per (32-K slab, pair of output columns n and n + 4 of an 8-column group): the two
// columns share their four weight words, so the thread writes whole words.  Per column and group of
// four K positions: keep the two largest magnitudes (ties: the higher index stays), quantise
// code = clamp(rint(fp16(w / s)) + 8, 0, 15), compress by the non-zero pattern of the kept codes with
// the selection table of sparsity.py:205-244 (a kept element whose code is 0 counts as pruned,
// exactly as in the reference), emit the two stored codes and the metadata nibble.
#pragma once

#include "common.cuh"

namespace trb {

// first | second << 2 for each non-zero pattern (bit i = element i of the group is non-zero).
__device__ __forceinline__ int select_nibble(int pat) {
  const bool m0 = pat & 1, m1 = pat & 2, m3 = pat & 8;
  const bool e0 = m0 && m1, e1 = !m0 && m1, e2 = !m0 && !m1;
  const int first = (int)e1 | ((int)e2 << 1);
  const int second = (int)(e0 || e2 || m3) | ((int)(e1 || !m1) << 1);
  return first | (second << 2);
}

// Flat int16 offset of nominal metadata element (row r of n_rows, column c): the row reorder
// inside 64-row groups and the 2 x 2 swizzle of sparsity.py:134-161.
__device__ __forceinline__ long long meta_offset(int r, int c, int n_rows) {
  int dst = (r / 64) * 64 + (r % 2) * 2 + (r % 8) / 4 + ((r % 32) % 4) / 2 * 32 + ((r % 64) / 8) * 4;
  const int tr = (dst % 2 == 0 && c % 2 == 1) ? 1 : 0;
  const int bl = (dst % 2 == 1 && c % 2 == 0) ? 1 : 0;
  dst += tr - bl;
  c += bl - tr;
  return (long long)(c / 2) * n_rows * 2 + (long long)dst * 2 + c % 2;
}

__global__ void pack_2_4_kernel(const __half* __restrict__ w, const __half* __restrict__ s_log,
                                uint32_t* __restrict__ q, int16_t* __restrict__ meta, __half* __restrict__ s_out,
                                int N, int K, int groups) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;   // column pair
  const int kt = blockIdx.y;                              // 32-K slab
  if (t >= N / 2) return;
  const int n0 = (t / 4) * 8 + (t % 4);                   // columns n0 and n0 + 4
  const int rows_per_group = K / groups;
  uint32_t words[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int n = n0 + 4 * h;
    const float sc = __half2float(s_log[(size_t)((kt * 32) / rows_per_group) * N + n]);
    int nominal[2] = {0, 0};
#pragma unroll
    for (int grp = 0; grp < 8; ++grp) {
      float mag[4];
      int code[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __half v = w[(size_t)(kt * 32 + grp * 4 + e) * N + n];
        mag[e] = fabsf(__half2float(v));
        const __half qv = __float2half_rn(__half2float(v) / sc);          // the fp16 quotient torch forms
        const int c = (int)rintf(__half2float(qv)) + 8;
        code[e] = c < 0 ? 0 : (c > 15 ? 15 : c);
      }
      // drop the two smallest magnitudes; among equals the lower index goes first
      int keep = 0xF;
#pragma unroll
      for (int round = 0; round < 2; ++round) {
        int lo = -1;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if ((keep >> e) & 1)
            if (lo < 0 || mag[e] < mag[lo]) lo = e;
        keep &= ~(1 << lo);
      }
      int pat = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (((keep >> e) & 1) && code[e] != 0) pat |= 1 << e;
      const int nib = select_nibble(pat);
      const int first = nib & 3, second = nib >> 2;
      int c_first = 0, c_second = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ce = ((keep >> e) & 1) ? code[e] : 0;
        if (e == first) c_first = ce;
        if (e == second) c_second = ce;
      }
      nominal[grp >> 2] |= nib << (4 * (grp & 3));
      // compressed rows 2 * grp and 2 * grp + 1 of the slab
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const int crow = 2 * grp + which;
        const int p = (crow / 8) + 2 * h + 4 * (crow % 2);
        words[(crow % 8) / 2] |= (uint32_t)(which ? c_second : c_first) << (4 * p);
      }
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) meta[meta_offset(n, 2 * kt + c, N)] = (int16_t)nominal[c];
    // stored scales: once per group (its first slab); every 8 columns stored as 0,4,1,5,2,6,3,7
    if ((kt * 32) % rows_per_group == 0) {
      const int g = (kt * 32) / rows_per_group;
      const int inv[8] = {0, 2, 4, 6, 1, 3, 5, 7};
      const int pos = groups == 1 ? n : (n & ~7) + inv[n & 7];
      s_out[(size_t)g * N + pos] = s_log[(size_t)g * N + n];
    }
  }
  // words of lanes i = 4 * (r / 8) + m, register j: word index blk * 128 + i * 4 + j
  const int blk = n0 / 64, r = n0 % 64, j = r % 4;
  uint32_t* row = q + (size_t)kt * 2 * N + blk * 128;
#pragma unroll
  for (int m = 0; m < 4; ++m) row[(4 * (r / 8) + m) * 4 + j] = words[m];
}

}  // namespace trb

extern "C" int trb_pack_2_4(const void* weight_kn, const void* scales_logical, void* qweight, void* meta,
                            void* scales_stored, int prob_k, int prob_m, int groupsize, int dev, void* stream) {
  using namespace trb;
  if (prob_k <= 0 || prob_m <= 0) return TRB_OK;
  if (!weight_kn || !scales_logical || !qweight || !meta || !scales_stored) return TRB_ERR_BAD_ARG;
  if (prob_k % 128 != 0 || prob_m % 256 != 0) return TRB_ERR_PROB_SHAPE;
  if (groupsize != -1 && groupsize != 128) return TRB_ERR_KERN_SHAPE;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  const int groups = groupsize == -1 ? 1 : prob_k / groupsize;
  dim3 grid((prob_m / 2 + 127) / 128, prob_k / 32);
  pack_2_4_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const __half*)weight_kn, (const __half*)scales_logical,
                                                          (uint32_t*)qweight, (int16_t*)meta, (__half*)scales_stored,
                                                          prob_m, prob_k, groups);
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}
