// Multi-GPU form of the indexed delta matmul: deltas are sharded by id over `world` ranks
// (owner = id % world, local id = id / world) and tokens travel to the owner and back through
// fixed-capacity exchange buffers, so that the collectives in between (all-to-all with equal splits,
// issued by the host through NCCL) need no counts on the host and no host synchronisation.
//
// Exchange buffer layout (both directions): `world` chunks, chunk r = rows for / from rank r,
// cap + 1 rows each.  Outbound chunk: rows 0..cap-1 = activation rows (K halves), row cap = the rows'
// local delta ids as int32, the number of rows in use, then each row's token row on the sender.  Return chunk: rows of N halves in
// the same slots.  The reference has no distributed layer; nothing here has a counterpart in it.
#pragma once

#include "common.cuh"
#include "route.cuh"

namespace trb {

// One CTA per token: copy its row into its slot of the send buffer and record its local delta id.
// CTAs T .. T + world - 1 write the per-chunk row counts.
// inline_plan: small batches skip the router launch; every CTA counts for itself how many earlier
// tokens go to the same rank (the same stable order the router gives) and writes slot_of.
__device__ __forceinline__ int block_sum_128(int v, int* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  const int total = sm[0] + sm[1] + sm[2] + sm[3];
  __syncthreads();
  return total;
}

__global__ void shard_pack_kernel(const uint4* __restrict__ x, const int* __restrict__ indices,
                                  int* __restrict__ slot_of, const int* __restrict__ bin_count,
                                  unsigned char* __restrict__ send, unsigned char* const* __restrict__ peers,
                                  int my_rank, uint4* __restrict__ y_zero, int N, int T, int K, int world, int cap,
                                  int inline_plan) {
  __shared__ int sm_cnt[4];
  // Chunk for rank r: in the local send buffer at chunk index r, or (peer mode) straight in rank r's
  // receive buffer at chunk index my_rank, written over NVLink.
  pdl_wait();   // slot_of and bin_count come from the router launched just before
  const long long row_bytes = (long long)K * 2;
  auto chunk = [&](int r) -> unsigned char* {
    return peers ? peers[r] + (long long)my_rank * (cap + 1) * row_bytes : send + (long long)r * (cap + 1) * row_bytes;
  };
  const int b = blockIdx.x;
  if (b >= T) {
    const int r = b - T;
    if (r >= world) return;
    int count;
    if (inline_plan) {
      int c = 0;
      for (int t = threadIdx.x; t < T; t += blockDim.x) {
        const int id = indices[t];
        c += (id >= 0 && id % world == r) ? 1 : 0;
      }
      count = block_sum_128(c, sm_cnt);
    } else {
      count = bin_count[r];
    }
    if (threadIdx.x == 0) {
      int* ids = reinterpret_cast<int*>(chunk(r) + (long long)cap * row_bytes);
      ids[cap] = min(count, cap);
    }
    return;
  }
  int slot;
  if (inline_plan) {
    const int my_id = indices[b];
    const int my_r = my_id >= 0 ? my_id % world : -1;
    int c = 0;
    for (int t = threadIdx.x; t < b; t += blockDim.x) {
      const int id = indices[t];
      c += (id >= 0 && id % world == my_r) ? 1 : 0;
    }
    const int q = block_sum_128(c, sm_cnt);
    slot = my_r >= 0 ? my_r * cap + q : -1;
    if (threadIdx.x == 0) slot_of[b] = slot;
  } else {
    slot = slot_of[b];
  }
  if (slot < 0) {
    // Peer form: nobody will write this token's output row, so it is cleared here.
    if (y_zero)
      for (int i = threadIdx.x; i < N / 8; i += blockDim.x) y_zero[(long long)b * (N / 8) + i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int r = slot / cap, q = slot - r * cap;
  if (r >= world) return;
  uint4* dst = reinterpret_cast<uint4*>(chunk(r) + (long long)q * row_bytes);
  const uint4* srcp = x + (long long)b * (K / 8);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = srcp[i];
  if (threadIdx.x == 0) {
    int* ids = reinterpret_cast<int*>(chunk(r) + (long long)cap * row_bytes);
    ids[q] = indices[b] / world;
    if ((long long)(2 * cap + 2) * 4 <= row_bytes) ids[cap + 1 + q] = b;   // the token's own row, for peer-form results
  }
}

// y[t] (+)= result row of token t's slot; tokens without a delta are zeroed unless accumulating.
__global__ void shard_combine_kernel(const uint4* __restrict__ back, const int* __restrict__ slot_of,
                                     uint4* __restrict__ y, int T, int N, int world, int cap, int accumulate) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const int slot = slot_of[t];
  uint4* dst = y + (long long)t * (N / 8);
  if (slot < 0) {
    if (!accumulate)
      for (int i = threadIdx.x; i < N / 8; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int r = slot / cap, q = slot - r * cap;
  const uint4* srcp = back + ((long long)r * (cap + 1) + q) * (N / 8);
  for (int i = threadIdx.x; i < N / 8; i += blockDim.x) {
    uint4 v = srcp[i];
    if (accumulate) {
      uint4 o = dst[i];
      __half2* vh = reinterpret_cast<__half2*>(&v);
      const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) vh[e] = __hadd2(vh[e], oh[e]);
    }
    dst[i] = v;
  }
}

}  // namespace trb

extern "C" size_t trb_shard_buffer_rows(int num_tokens, int world) {
  return (num_tokens <= 0 || world <= 0) ? 0 : (size_t)world * ((size_t)num_tokens + 1);
}

// Plan + pack: slot_of[T] (out), send buffer [world][T + 1][K] halves (out).  plan: int32 [8 + world].
extern "C" int trb_shard_dispatch(const void* x, const void* indices, int num_tokens, int prob_k, int world,
                                  void* send_buf, const void* peer_recv_ptrs, int my_rank, void* y_zero, int prob_m,
                                  void* slot_of, void* plan, int dev, void* stream_v) {
  using namespace trb;
  cudaStream_t stream = (cudaStream_t)stream_v;
  if (num_tokens == 0) return TRB_OK;
  if (num_tokens < 0 || world < 1 || world > 64 || prob_k <= 0 || prob_k % 8 != 0) return TRB_ERR_BAD_ARG;
  if (!x || !indices || (!send_buf && !peer_recv_ptrs) || !slot_of || !plan) return TRB_ERR_BAD_ARG;
  if (my_rank < 0 || my_rank >= world) return TRB_ERR_BAD_ARG;
  if ((long long)num_tokens * 4 + 4 > (long long)prob_k * 2) return TRB_ERR_PROB_SHAPE;  // ids must fit one row
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  int* counters = (int*)plan;
  int* bin_count = counters + 8;
  RouteSrc src{};
  src.indices = (const int*)indices;
  src.mod = world;
  // Small batches plan inside the pack kernel (one launch less); large ones go through the router.
  const int inline_plan = num_tokens <= 1024 ? 1 : 0;
  if (!inline_plan) {
    const int rc = route_launch_src(src, num_tokens, world, 1 << 30, nullptr, nullptr, nullptr, nullptr, nullptr,
                                    nullptr, nullptr, counters, (int*)slot_of, num_tokens, bin_count, stream);
    if (rc != TRB_OK) return rc;
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(num_tokens + world);
  lc.blockDim = dim3(128);
  lc.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits (pdl_wait) before it reads
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return cudaLaunchKernelEx(&lc, shard_pack_kernel, (const uint4*)x, (const int*)indices, (int*)slot_of,
                            (const int*)bin_count, (unsigned char*)send_buf, (unsigned char* const*)peer_recv_ptrs,
                            my_rank, (uint4*)y_zero, prob_m, num_tokens, prob_k, world, num_tokens,
                            inline_plan) == cudaSuccess
             ? TRB_OK
             : TRB_ERR_CUDA;
}

extern "C" int trb_shard_combine(const void* back_buf, const void* slot_of, void* y, int num_tokens, int prob_m,
                                 int world, int accumulate, int dev, void* stream_v) {
  using namespace trb;
  if (num_tokens == 0) return TRB_OK;
  if (num_tokens < 0 || world < 1 || prob_m <= 0 || prob_m % 8 != 0 || !back_buf || !slot_of || !y)
    return TRB_ERR_BAD_ARG;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  shard_combine_kernel<<<num_tokens, 128, 0, (cudaStream_t)stream_v>>>((const uint4*)back_buf, (const int*)slot_of,
                                                                      (uint4*)y, num_tokens, prob_m, world,
                                                                      num_tokens, accumulate);
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}
