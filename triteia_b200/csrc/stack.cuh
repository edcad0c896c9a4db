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
