// On-GPU decoder of the packed int4 + 2:4 format: dense fp16 W[K, N] from (qweight, meta, scales).
// One thread per (32-K slab, output column): 16 stored codes from four weight words, two
// metadata half-words, W = fp16(code - 8) * fp16(scale) rounded once.  Format references:
// triteia/python/nn/linear.py:128-138 (nibble placement), triteia/python/ops/utils/sparsity.py
// :35-54 (lane permutation), :134-161 (metadata order), :246-272 (metadata nibble meaning).
#pragma once

#include "common.cuh"

namespace trb {

__global__ void unpack_2_4_kernel(const uint32_t* __restrict__ q, const uint16_t* __restrict__ meta,
                                  const __half* __restrict__ s, __half* __restrict__ w, int N, int K, int grouped) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int kt = blockIdx.y;
  if (n >= N) return;
  const int blk = n >> 6, r = n & 63;
  const int g = r >> 3, within = r & 7, block = within >> 2, j = within & 3;
  // Physical metadata row of output column n inside its 64-row group, and the half-word that
  // holds it: word (row & ~1) + c carries dense positions 16c..16c+15 of the slab.
  const int mrow = (r & 1) * 2 + (r & 7) / 4 + ((r & 31) & 3) / 2 * 32 + (r >> 3) * 4;
  const uint16_t* mslab = meta + ((size_t)kt * N + blk * 64) * 2;
  uint32_t mbits = 0;  // 8 nibbles: groups 0..7 of the slab
#pragma unroll
  for (int c = 0; c < 2; ++c) mbits |= (uint32_t)mslab[((mrow & ~1) + c) * 2 + (mrow & 1)] << (16 * c);

  __half sc;
  if (grouped) {
    const int pos = (within < 4) ? 2 * within : 2 * (within - 4) + 1;  // stored order 0,4,1,5,2,6,3,7
    sc = s[(size_t)(kt >> 2) * N + (n & ~7) + pos];
  } else {
    sc = s[n];
  }
  __half out[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) out[i] = __float2half(0.f);
  const uint32_t* qrow = q + (size_t)kt * 2 * N + blk * 128;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const uint32_t word = qrow[(4 * g + m) * 4 + j];
#pragma unroll
    for (int hi8 = 0; hi8 < 2; ++hi8)
#pragma unroll
      for (int hi1 = 0; hi1 < 2; ++hi1) {
        const int p = hi1 * 4 + block * 2 + hi8;
        const int code = (word >> (4 * p)) & 15;
        const int crow = 2 * m + hi1 + 8 * hi8;      // compressed row inside the slab
        const int grp = crow >> 1, which = crow & 1;
        const int nib = (mbits >> (4 * grp)) & 15;
        const int pos = which ? (nib >> 2) & 3 : nib & 3;
        out[4 * grp + pos] = __hmul(__int2half_rn(code - 8), sc);
      }
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) w[(size_t)(kt * 32 + i) * N + n] = out[i];
}

}  // namespace trb

extern "C" int trb_unpack_2_4(const void* B, const void* meta, const void* s, void* w_out, int prob_m, int prob_k,
                              int groupsize, int dev, void* stream) {
  using namespace trb;
  if (prob_m <= 0 || prob_k <= 0) return TRB_OK;
  if (!B || !meta || !s || !w_out) return TRB_ERR_BAD_ARG;
  if (prob_m % 64 != 0 || prob_k % 128 != 0) return TRB_ERR_PROB_SHAPE;
  if (groupsize != -1 && groupsize != 128) return TRB_ERR_KERN_SHAPE;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  dim3 grid((prob_m + 127) / 128, prob_k / 32);
  unpack_2_4_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const uint32_t*)B, (const uint16_t*)meta,
                                                            (const __half*)s, (__half*)w_out, prob_m, prob_k,
                                                            groupsize == 128);
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}
