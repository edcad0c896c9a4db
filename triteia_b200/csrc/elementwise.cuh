// Element-wise neighbours of the linears in a decoder layer, as the reference's extension module
// offers them: gelu_quick (triteia/csrc/ops/activations.cu:181-207), silu_and_mul
// (activations.cu:14-78) and rotary_embedding (triteia/csrc/ops/pos_encoding_kernels.cu:10-130).
// HBM-bound: 16-byte accesses for the activations, one CTA per token for the rotation.
#pragma once

#include "common.cuh"

namespace trb {

template <class T>
struct Ew;
template <>
struct Ew<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <>
struct Ew<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// out[i] = x / (1 + exp(-1.702 x)), the result rounded once from fp32.
template <class T>
__global__ void gelu_quick_kernel(T* __restrict__ out, const T* __restrict__ in, long long n_vec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
    uint4 v = reinterpret_cast<const uint4*>(in)[i];
    T* e = reinterpret_cast<T*>(&v);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float x = Ew<T>::to_f(e[k]);
      e[k] = Ew<T>::from_f(x / (1.0f + expf(-1.702f * x)));
    }
    reinterpret_cast<uint4*>(out)[i] = v;
  }
}

// out[t, i] = silu(in[t, i]) * in[t, d + i]; silu rounded to T before the product, as the reference
// computes it (ACT_FN returns scalar_t, then scalar_t * scalar_t).
template <class T>
__global__ void silu_and_mul_kernel(T* __restrict__ out, const T* __restrict__ in, int d_vec) {
  const long long t = blockIdx.x;
  const uint4* g = reinterpret_cast<const uint4*>(in) + t * 2 * d_vec;
  const uint4* u = g + d_vec;
  uint4* o = reinterpret_cast<uint4*>(out) + t * d_vec;
  for (int i = threadIdx.x; i < d_vec; i += blockDim.x) {
    uint4 a = g[i];
    const uint4 b = u[i];
    T* ae = reinterpret_cast<T*>(&a);
    const T* be = reinterpret_cast<const T*>(&b);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float x = Ew<T>::to_f(ae[k]);
      const T act = Ew<T>::from_f(x / (1.0f + expf(-x)));
      ae[k] = Ew<T>::from_f(Ew<T>::to_f(act) * Ew<T>::to_f(be[k]));
    }
    o[i] = a;
  }
}

// In-place rotation of the first rot_dim elements of every head of query and key.  One CTA per
// token; cos_sin_cache row `pos (+ offset)`: rot_dim / 2 cosines then rot_dim / 2 sines.
// NEOX pairs element i with i + rot_dim / 2, GPT-J pairs 2i with 2i + 1.  fp32 arithmetic, one rounding.
template <class T, bool NEOX>
__global__ void rotary_kernel(const int64_t* __restrict__ positions, T* __restrict__ query, T* __restrict__ key,
                              const T* __restrict__ cache, const int64_t* __restrict__ offsets, int rot_dim,
                              long long q_stride, long long k_stride, int num_heads, int num_kv_heads, int head_size) {
  const long long t = blockIdx.x;
  const long long row = positions[t] + (offsets ? offsets[t] : 0);
  const T* cos_p = cache + row * rot_dim;
  const int embed = rot_dim / 2;
  const T* sin_p = cos_p + embed;
  const int nq = num_heads * embed, nk = key ? num_kv_heads * embed : 0;
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
    const bool is_q = i < nq;
    const int ii = is_q ? i : i - nq;
    const int head = ii / embed, off = ii - head * embed;
    T* arr = (is_q ? query + t * q_stride : key + t * k_stride) + (long long)head * head_size;
    const int xi = NEOX ? off : 2 * off, yi = NEOX ? embed + off : 2 * off + 1;
    const float c = Ew<T>::to_f(cos_p[off]), s = Ew<T>::to_f(sin_p[off]);
    const float x = Ew<T>::to_f(arr[xi]), y = Ew<T>::to_f(arr[yi]);
    arr[xi] = Ew<T>::from_f(x * c - y * s);
    arr[yi] = Ew<T>::from_f(y * c + x * s);
  }
}

}  // namespace trb

extern "C" int trb_gelu_quick(void* out, const void* in, long long numel, int dtype, int dev, void* stream) {
  using namespace trb;
  if (numel == 0) return TRB_OK;
  if (numel < 0 || !out || !in) return TRB_ERR_BAD_ARG;
  if (numel % 8 != 0 || (((uintptr_t)out | (uintptr_t)in) & 15)) return TRB_ERR_PROB_SHAPE;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  const long long n_vec = numel / 8;
  const int grid = (int)((n_vec + 255) / 256 < 148 * 8 ? (n_vec + 255) / 256 : 148 * 8);
  if (dtype == TRB_F16)
    gelu_quick_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((__half*)out, (const __half*)in, n_vec);
  else if (dtype == TRB_BF16)
    gelu_quick_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)in, n_vec);
  else
    return TRB_ERR_KERN_SHAPE;
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}

extern "C" int trb_silu_and_mul(void* out, const void* in, int num_tokens, int d, int dtype, int dev, void* stream) {
  using namespace trb;
  if (num_tokens == 0 || d == 0) return TRB_OK;
  if (num_tokens < 0 || d < 0 || !out || !in) return TRB_ERR_BAD_ARG;
  if (d % 8 != 0 || (((uintptr_t)out | (uintptr_t)in) & 15)) return TRB_ERR_PROB_SHAPE;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  const int threads = d / 8 < 256 ? ((d / 8 + 31) / 32) * 32 : 256;
  if (dtype == TRB_F16)
    silu_and_mul_kernel<__half><<<num_tokens, threads, 0, (cudaStream_t)stream>>>((__half*)out, (const __half*)in, d / 8);
  else if (dtype == TRB_BF16)
    silu_and_mul_kernel<__nv_bfloat16><<<num_tokens, threads, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)in, d / 8);
  else
    return TRB_ERR_KERN_SHAPE;
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}

extern "C" int trb_rotary_embedding(const void* positions, void* query, void* key, const void* cos_sin_cache,
                                    const void* cache_offsets, int num_tokens, int rot_dim, long long query_stride,
                                    long long key_stride, int num_heads, int num_kv_heads, int head_size, int is_neox,
                                    int dtype, int dev, void* stream) {
  using namespace trb;
  if (num_tokens == 0) return TRB_OK;
  if (num_tokens < 0 || !positions || !query || !cos_sin_cache) return TRB_ERR_BAD_ARG;
  if (rot_dim <= 0 || rot_dim % 2 != 0 || rot_dim > head_size || num_heads <= 0 || num_kv_heads < 0) return TRB_ERR_PROB_SHAPE;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  const int work = num_heads * rot_dim / 2;
  const int threads = work < 512 ? ((work + 31) / 32) * 32 : 512;
  cudaStream_t st = (cudaStream_t)stream;
#define TRB_ROTARY(T, NEOX)                                                                                          \
  rotary_kernel<T, NEOX><<<num_tokens, threads, 0, st>>>((const int64_t*)positions, (T*)query, (T*)key,              \
                                                         (const T*)cos_sin_cache, (const int64_t*)cache_offsets,      \
                                                         rot_dim, query_stride, key_stride, num_heads, num_kv_heads, \
                                                         head_size)
  if (dtype == TRB_F16) {
    if (is_neox) TRB_ROTARY(__half, true); else TRB_ROTARY(__half, false);
  } else if (dtype == TRB_BF16) {
    if (is_neox) TRB_ROTARY(__nv_bfloat16, true); else TRB_ROTARY(__nv_bfloat16, false);
  } else {
    return TRB_ERR_KERN_SHAPE;
  }
#undef TRB_ROTARY
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}
