// LoRA operators of the path: BGMV (one adapter per token, mat-vec), a fused shrink->expand
// variant that keeps the rank-r intermediate on chip, and SGMV (one adapter per contiguous token
// segment, small tensor-core GEMMs).  Semantics follow the reference's Punica-derived kernels:
// triteia/csrc/ops/bgmv_impl.cuh:15-207 (shrink / expand), triteia/csrc/ops/sgmv.cuh:61-174
// (grouped GEMM with alpha = beta = 1, fp32 accumulation) and the docstrings of
// triteia/python/capi/punica.py:13-27,43-60.  All launches go to the caller's stream.
#pragma once

#include "common.cuh"

namespace trb {

template <class T> struct Cvt;
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float2 to_f2(uint32_t v) { return __half22float2(*reinterpret_cast<__half2*>(&v)); }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float2 to_f2(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
  }
};

template <class T>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
  const uint32_t* pa = reinterpret_cast<const uint32_t*>(&a);
  const uint32_t* pb = reinterpret_cast<const uint32_t*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = Cvt<T>::to_f2(pa[i]), fb = Cvt<T>::to_f2(pb[i]);
    s = fmaf(fa.x, fb.x, s);
    s = fmaf(fa.y, fb.y, s);
  }
  return s;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- BGMV, long dot products (h_in >= 256): one warp per output feature ----
template <class T>
__global__ void bgmv_long_kernel(T* __restrict__ Y, const T* __restrict__ X, const T* __restrict__ W,
                                 const int64_t* __restrict__ indices, int h_in, int h_out, int num_layers,
                                 int layer_idx, float scale) {
  const int b = blockIdx.y;
  const int o = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (o >= h_out) return;
  const int64_t idx = indices[b];
  if (idx < 0) return;
  const uint4* w = reinterpret_cast<const uint4*>(W + ((idx * num_layers + layer_idx) * h_out + o) * (int64_t)h_in);
  const uint4* x = reinterpret_cast<const uint4*>(X + (int64_t)b * h_in);
  float s = 0.f;
  for (int i = lane; i < h_in / 8; i += 32) s += dot8<T>(w[i], x[i]);
  s = warp_sum(s);
  if (lane == 0) {
    T* y = Y + (int64_t)b * h_out + o;
    *y = Cvt<T>::from_f(Cvt<T>::to_f(*y) + scale * s);
  }
}

// ---- BGMV, short dot products (h_in < 256, i.e. the rank): one thread per output feature ----
template <class T>
__global__ void bgmv_short_kernel(T* __restrict__ Y, const T* __restrict__ X, const T* __restrict__ W,
                                  const int64_t* __restrict__ indices, int h_in, int h_out, int num_layers,
                                  int layer_idx, float scale) {
  __shared__ uint4 xs[32];
  const int b = blockIdx.y;
  const int64_t idx = indices[b];
  if (idx < 0) return;
  const int nv = h_in / 8;
  if (threadIdx.x < nv) xs[threadIdx.x] = reinterpret_cast<const uint4*>(X + (int64_t)b * h_in)[threadIdx.x];
  __syncthreads();
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= h_out) return;
  const uint4* w = reinterpret_cast<const uint4*>(W + ((idx * num_layers + layer_idx) * h_out + o) * (int64_t)h_in);
  float s = 0.f;
  for (int i = 0; i < nv; ++i) s += dot8<T>(w[i], xs[i]);
  T* y = Y + (int64_t)b * h_out + o;
  *y = Cvt<T>::from_f(Cvt<T>::to_f(*y) + scale * s);
}

// ---- fused decode LoRA: one CTA per token, v = A^T x kept in shared memory ----
template <class T>
__global__ void __launch_bounds__(256) lora_fused_kernel(T* __restrict__ Y, const T* __restrict__ X,
                                                         const T* __restrict__ WA, const T* __restrict__ WB,
                                                         const int64_t* __restrict__ indices, int h1, int h2,
                                                         int rank, int num_layers, int layer_idx, float scale) {
  extern __shared__ uint4 xsm[];   // x row: h1 / 8 vectors
  __shared__ float v[64];
  const int b = blockIdx.x;
  const int64_t idx = indices[b];
  if (idx < 0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nv = h1 / 8;
  const uint4* x = reinterpret_cast<const uint4*>(X + (int64_t)b * h1);
  for (int i = tid; i < nv; i += 256) xsm[i] = x[i];
  __syncthreads();
  const T* wa = WA + (idx * num_layers + layer_idx) * (int64_t)rank * h1;
  for (int j = warp; j < rank; j += 8) {
    const uint4* row = reinterpret_cast<const uint4*>(wa + (int64_t)j * h1);
    float s = 0.f;
    for (int i = lane; i < nv; i += 32) s += dot8<T>(row[i], xsm[i]);
    s = warp_sum(s);
    if (lane == 0) v[j] = s * scale;
  }
  __syncthreads();
  const T* wb = WB + (idx * num_layers + layer_idx) * (int64_t)h2 * rank;
  const int rv = rank / 8;
  for (int o = tid; o < h2; o += 256) {
    const uint4* row = reinterpret_cast<const uint4*>(wb + (int64_t)o * rank);
    float s = 0.f;
    for (int i = 0; i < rv; ++i) {
      const uint4 wv = row[i];
      const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = Cvt<T>::to_f2(pw[e]);
        s = fmaf(f.x, v[i * 8 + 2 * e], s);
        s = fmaf(f.y, v[i * 8 + 2 * e + 1], s);
      }
    }
    T* y = Y + (int64_t)b * h2 + o;
    *y = Cvt<T>::from_f(Cvt<T>::to_f(*y) + s);
  }
}

// ---- indexed LoRA on the natural layouts A [M, h1, r], B [M, r, h2]: one CTA per token ----
// The id space may be shared with deltas: ids outside [0, num_adapters) are skipped.
template <class T, class IdxT>
__global__ void __launch_bounds__(256) lora_indexed_kernel(T* __restrict__ Y, const T* __restrict__ X,
                                                           const T* __restrict__ A, const T* __restrict__ B,
                                                           const IdxT* __restrict__ indices, int h1, int h2, int rank,
                                                           int num_adapters, float scale) {
  __shared__ float part[8][64];
  __shared__ float v[64];
  const int b = blockIdx.x;
  const long long idx = (long long)indices[b];
  if (idx < 0 || idx >= num_adapters) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* a = A + idx * (int64_t)h1 * rank;
  const T* x = X + (int64_t)b * h1;
  float acc[64];
#pragma unroll
  for (int j = 0; j < 64; ++j) acc[j] = 0.f;
  const int rv = rank / 8;
  for (int k = tid; k < h1; k += 256) {
    const float xk = Cvt<T>::to_f(x[k]);
    const uint4* row = reinterpret_cast<const uint4*>(a + (int64_t)k * rank);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i < rv) {
        const uint4 wv = row[i];
        const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = Cvt<T>::to_f2(pw[e]);
          acc[i * 8 + 2 * e] = fmaf(xk, f.x, acc[i * 8 + 2 * e]);
          acc[i * 8 + 2 * e + 1] = fmaf(xk, f.y, acc[i * 8 + 2 * e + 1]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 64; ++j) {
    if (j < rank) {
      const float s = warp_sum(acc[j]);
      if (lane == 0) part[warp][j] = s;
    }
  }
  __syncthreads();
  if (tid < rank) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += part[w][tid];
    v[tid] = s * scale;
  }
  __syncthreads();
  const T* bm = B + idx * (int64_t)rank * h2;
  for (int o8 = tid; o8 < h2 / 8; o8 += 256) {
    float out[8];
    const uint4 yv = *reinterpret_cast<const uint4*>(Y + (int64_t)b * h2 + o8 * 8);
    const uint32_t* py = reinterpret_cast<const uint32_t*>(&yv);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = Cvt<T>::to_f2(py[e]);
      out[2 * e] = f.x;
      out[2 * e + 1] = f.y;
    }
    for (int j = 0; j < rank; ++j) {
      const uint4 wv = *reinterpret_cast<const uint4*>(bm + (int64_t)j * h2 + o8 * 8);
      const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv);
      const float vj = v[j];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = Cvt<T>::to_f2(pw[e]);
        out[2 * e] = fmaf(vj, f.x, out[2 * e]);
        out[2 * e + 1] = fmaf(vj, f.y, out[2 * e + 1]);
      }
    }
    T o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = Cvt<T>::from_f(out[e]);
    *reinterpret_cast<uint4*>(Y + (int64_t)b * h2 + o8 * 8) = *reinterpret_cast<uint4*>(o);
  }
}

// ---- SGMV: y[seg] += x[seg] @ W_seg, 64-token x BN-column tiles on mma.sync m16n8k16 ----
// grid = (column tiles, token-tile lanes, problems); each CTA walks the token tiles of its problem
// with stride gridDim.y.  K runs through a 3-stage cp.async ring of 64-deep slices; fragments come
// from ldmatrix (x4 for the token rows, x2.trans for the row-major weight slice).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;   // zero-fill when the source is out of range
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr) : "memory");
}

template <int BN>
struct SgmvSmem {
  static constexpr int BK = 64, STAGES = 3;
  static constexpr int XLD = BK + 8, WLD = BN + 8;              // halves; +8 keeps ldmatrix rows on distinct banks
  static constexpr int X_BYTES = 64 * XLD * 2, W_BYTES = BK * WLD * 2;
  static constexpr int STAGE_BYTES = X_BYTES + W_BYTES;
  static constexpr int BYTES = STAGES * STAGE_BYTES;
};

template <class T, int BN>
__global__ void __launch_bounds__(128) sgmv_kernel(T* __restrict__ Y, const T* __restrict__ X,
                                                   const T* const* __restrict__ Wp, const int32_t* __restrict__ seg,
                                                   int d_in, int d_out, int layer_idx) {
  using SM = SgmvSmem<BN>;
  constexpr int BK = SM::BK, STAGES = SM::STAGES;
  extern __shared__ __align__(16) uint8_t sgmv_smem[];
  const uint32_t sbase = smem_u32(sgmv_smem);
  const int prob = blockIdx.z;
  const int r0 = max(0, seg[prob]), r1 = seg[prob + 1];
  const int col_base = blockIdx.x * BN;
  const T* W = Wp[prob] + (int64_t)layer_idx * d_in * d_out;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, m = lane & 3;
  const int k_slices = (d_in + BK - 1) / BK;

  for (int row_base = r0 + blockIdx.y * 64; row_base < r1; row_base += gridDim.y * 64) {
    auto load_slice = [&](int ks, int stage) {
      const int k0 = ks * BK;
      const uint32_t xs = sbase + stage * SM::STAGE_BYTES, ws = xs + SM::X_BYTES;
      for (int v = tid; v < 64 * (BK / 8); v += 128) {
        const int r = v / (BK / 8), c = (v % (BK / 8)) * 8;
        const bool ok = row_base + r < r1 && k0 + c < d_in;
        cp_async16(xs + (r * SM::XLD + c) * 2, ok ? (const void*)(X + (int64_t)(row_base + r) * d_in + k0 + c) : (const void*)X, ok);
      }
      for (int v = tid; v < BK * (BN / 8); v += 128) {
        const int r = v / (BN / 8), c = (v % (BN / 8)) * 8;
        const bool ok = k0 + r < d_in && col_base + c < d_out;
        cp_async16(ws + (r * SM::WLD + c) * 2, ok ? (const void*)(W + (int64_t)(k0 + r) * d_out + col_base + c) : (const void*)W, ok);
      }
    };
    float acc[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;

#pragma unroll
    for (int p = 0; p < STAGES - 1; ++p) {
      if (p < k_slices) load_slice(p, p);
      cp_async_commit();
    }
    for (int ks = 0; ks < k_slices; ++ks) {
      cp_async_wait<STAGES - 2>();
      __syncthreads();
      if (ks + STAGES - 1 < k_slices) load_slice(ks + STAGES - 1, (ks + STAGES - 1) % STAGES);
      cp_async_commit();
      const uint32_t xs = sbase + (ks % STAGES) * SM::STAGE_BYTES, ws = xs + SM::X_BYTES;
#pragma unroll
      for (int kk = 0; kk < BK; kk += 16) {
        uint32_t af[4];
        // rows warp*16 + (lane % 16), k offset kk + 8 * (lane / 16): matrices (r0-7,k0-7),(r8-15,k0-7),(r0-7,k8-15),(r8-15,k8-15)
        ldmatrix_x4(af, xs + ((warp * 16 + (lane & 15)) * SM::XLD + kk + 8 * (lane >> 4)) * 2);
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
          uint32_t b0, b1;
          // weight slice rows kk + (lane % 16), columns nt*8..+7, transposed on load
          ldmatrix_x2_trans(b0, b1, ws + ((kk + (lane & 15)) * SM::WLD + nt * 8) * 2);
          if constexpr (std::is_same<T, __half>::value) mma_m16n8k16(acc[nt], af, b0, b1);
          else mma_m16n8k16_bf16(acc[nt], af, b0, b1);
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();
    // Epilogue through shared memory (the pipeline's buffers are free now): the fp32 tile goes out
    // as [64 rows][BN columns], then every thread adds 8-column pieces of it into y with one 16-byte
    // read and one 16-byte write, rounding once (the accumulator fragment layout would touch
    // 16 bytes per row and instruction).
    constexpr int OLD = BN + 4;                      // padded row, in floats
    static_assert(64 * OLD * 4 <= SM::BYTES, "the output tile fits the pipeline's shared memory");
    float* otile = reinterpret_cast<float*>(sgmv_smem);
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
        *reinterpret_cast<float2*>(otile + (warp * 16 + g + 8 * h) * OLD + nt * 8 + 2 * m) =
            make_float2(acc[nt][2 * h], acc[nt][2 * h + 1]);
    }
    __syncthreads();
    for (int v = tid; v < 64 * (BN / 8); v += 128) {
      const int r = v / (BN / 8), c = (v % (BN / 8)) * 8;
      const int row = row_base + r, col = col_base + c;
      if (row < r1 && col < d_out) {
        uint4* yp = reinterpret_cast<uint4*>(Y + (int64_t)row * d_out + col);
        uint4 old = *yp;
        const float4 a0 = *reinterpret_cast<const float4*>(otile + r * OLD + c);
        const float4 a1 = *reinterpret_cast<const float4*>(otile + r * OLD + c + 4);
        const float add[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        uint32_t* ow = reinterpret_cast<uint32_t*>(&old);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 o = Cvt<T>::to_f2(ow[e]);
          T o2[2] = {Cvt<T>::from_f(o.x + add[2 * e]), Cvt<T>::from_f(o.y + add[2 * e + 1])};
          ow[e] = *reinterpret_cast<uint32_t*>(o2);
        }
        *yp = old;
      }
    }
    __syncthreads();                                 // the next tile's loads reuse this memory
  }  // token tiles
}

template <class T>
static int bgmv_launch(void* Y, const void* X, const void* W, const void* idx, int batch, int h_in, int h_out,
                       int num_layers, int layer_idx, float scale, cudaStream_t st) {
  if (h_in >= 256) {
    dim3 grid((h_out + 3) / 4, batch);
    bgmv_long_kernel<T><<<grid, 128, 0, st>>>((T*)Y, (const T*)X, (const T*)W, (const int64_t*)idx, h_in, h_out,
                                               num_layers, layer_idx, scale);
  } else {
    dim3 grid((h_out + 255) / 256, batch);
    bgmv_short_kernel<T><<<grid, 256, 0, st>>>((T*)Y, (const T*)X, (const T*)W, (const int64_t*)idx, h_in, h_out,
                                                num_layers, layer_idx, scale);
  }
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}

template <class T, int BN>
static void sgmv_launch_bn(void* y, const void* x, const void* w, const void* s, int num_problems, int d_in,
                           int d_out, int layer_idx, cudaStream_t st) {
  const int col_tiles = (d_out + BN - 1) / BN;
  int gy = (4 * 148 + col_tiles * num_problems - 1) / (col_tiles * num_problems);
  gy = gy < 1 ? 1 : (gy > 64 ? 64 : gy);
  dim3 grid(col_tiles, gy, num_problems);
  if (SgmvSmem<BN>::BYTES > 48 * 1024)
    cudaFuncSetAttribute(sgmv_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SgmvSmem<BN>::BYTES);
  sgmv_kernel<T, BN><<<grid, 128, SgmvSmem<BN>::BYTES, st>>>((T*)y, (const T*)x, (const T* const*)w, (const int32_t*)s, d_in, d_out,
                                            layer_idx);
}

template <class T>
static int sgmv_launch(void* y, const void* x, const void* w, const void* s, int num_problems, int d_in, int d_out,
                       int layer_idx, cudaStream_t st) {
  if (d_out <= 16) sgmv_launch_bn<T, 16>(y, x, w, s, num_problems, d_in, d_out, layer_idx, st);
  else if (d_out <= 32) sgmv_launch_bn<T, 32>(y, x, w, s, num_problems, d_in, d_out, layer_idx, st);
  else if (d_out <= 64) sgmv_launch_bn<T, 64>(y, x, w, s, num_problems, d_in, d_out, layer_idx, st);
  else sgmv_launch_bn<T, 128>(y, x, w, s, num_problems, d_in, d_out, layer_idx, st);
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}

}  // namespace trb

extern "C" int trb_bgmv(void* Y, const void* X, const void* W, const void* indices, int batch, int h_in, int h_out,
                        int num_layers, int layer_idx, float scale, int dtype, int dev, void* stream) {
  using namespace trb;
  if (batch == 0) return TRB_OK;
  if (batch < 0 || !Y || !X || !W || !indices || layer_idx < 0 || layer_idx >= num_layers) return TRB_ERR_BAD_ARG;
  if (h_in <= 0 || h_out <= 0 || h_in >= 65536 || h_out >= 65536 || h_in % 8 != 0) return TRB_ERR_KERN_SHAPE;
  if (batch > 65535) return TRB_ERR_KERN_SHAPE;
  if (((uintptr_t)X | (uintptr_t)W) & 15) return TRB_ERR_BAD_ARG;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  if (dtype == TRB_F16)
    return bgmv_launch<__half>(Y, X, W, indices, batch, h_in, h_out, num_layers, layer_idx, scale, (cudaStream_t)stream);
  if (dtype == TRB_BF16)
    return bgmv_launch<__nv_bfloat16>(Y, X, W, indices, batch, h_in, h_out, num_layers, layer_idx, scale,
                                      (cudaStream_t)stream);
  return TRB_ERR_KERN_SHAPE;
}

extern "C" int trb_lora_bgmv_fused(void* y, const void* x, const void* wa_t, const void* wb_t, const void* indices,
                                   int batch, int h1, int h2, int rank, int num_layers, int layer_idx, float scale,
                                   int dtype, int dev, void* stream) {
  using namespace trb;
  if (batch == 0) return TRB_OK;
  if (batch < 0 || !y || !x || !wa_t || !wb_t || !indices || layer_idx < 0 || layer_idx >= num_layers)
    return TRB_ERR_BAD_ARG;
  if (rank <= 0 || rank > 64 || rank % 8 != 0 || h1 % 8 != 0 || h1 <= 0 || h2 <= 0 || h1 > 65536)
    return TRB_ERR_KERN_SHAPE;
  if (((uintptr_t)x | (uintptr_t)wa_t | (uintptr_t)wb_t) & 15) return TRB_ERR_BAD_ARG;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  const size_t smem = (size_t)h1 * 2;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TRB_F16) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(lora_fused_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
      return TRB_ERR_CUDA;
    lora_fused_kernel<__half><<<batch, 256, smem, st>>>((__half*)y, (const __half*)x, (const __half*)wa_t,
                                                        (const __half*)wb_t, (const int64_t*)indices, h1, h2, rank,
                                                        num_layers, layer_idx, scale);
  } else if (dtype == TRB_BF16) {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(lora_fused_kernel<__nv_bfloat16>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return TRB_ERR_CUDA;
    lora_fused_kernel<__nv_bfloat16><<<batch, 256, smem, st>>>(
        (__nv_bfloat16*)y, (const __nv_bfloat16*)x, (const __nv_bfloat16*)wa_t, (const __nv_bfloat16*)wb_t,
        (const int64_t*)indices, h1, h2, rank, num_layers, layer_idx, scale);
  } else {
    return TRB_ERR_KERN_SHAPE;
  }
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}

extern "C" size_t trb_sgmv_tmp_size(int num_problems) {
  // Same size rule as the reference (three pointer arrays, three leading-dimension arrays and
  // one 12-byte problem shape per problem); the buffer itself is not used.
  return num_problems > 0 ? (size_t)num_problems * (3 * 8 + 3 * 8 + 12) : 0;
}

extern "C" int trb_sgmv(void* y, const void* x, const void* w, const void* s, void* tmp, int num_problems, int d_in,
                        int d_out, int layer_idx, int dtype, int dev, void* stream) {
  using namespace trb;
  (void)tmp;
  if (num_problems == 0) return TRB_OK;
  if (num_problems < 0 || !y || !x || !w || !s || layer_idx < 0) return TRB_ERR_BAD_ARG;
  if (d_in <= 0 || d_out <= 0 || d_in % 8 != 0 || d_out % 8 != 0 || num_problems > 65535) return TRB_ERR_KERN_SHAPE;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  if (((uintptr_t)x | (uintptr_t)y) & 15) return TRB_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TRB_F16) return sgmv_launch<__half>(y, x, w, s, num_problems, d_in, d_out, layer_idx, st);
  if (dtype == TRB_BF16) return sgmv_launch<__nv_bfloat16>(y, x, w, s, num_problems, d_in, d_out, layer_idx, st);
  return TRB_ERR_KERN_SHAPE;
}

extern "C" int trb_lora_indexed(void* y, const void* x, const void* wa, const void* wb, const void* indices,
                                int index_is_64bit, int batch, int h1, int h2, int rank, int num_adapters,
                                float scale, int dtype, int dev, void* stream) {
  using namespace trb;
  if (batch == 0 || num_adapters == 0) return TRB_OK;
  if (batch < 0 || num_adapters < 0 || !y || !x || !wa || !wb || !indices) return TRB_ERR_BAD_ARG;
  if (rank <= 0 || rank > 64 || rank % 8 != 0 || h1 <= 0 || h2 <= 0 || h2 % 8 != 0) return TRB_ERR_KERN_SHAPE;
  if (((uintptr_t)y | (uintptr_t)wa | (uintptr_t)wb) & 15) return TRB_ERR_BAD_ARG;
  if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
  cudaStream_t st = (cudaStream_t)stream;
#define TRB_LORA_IDX(T, I)                                                                                        \
  lora_indexed_kernel<T, I><<<batch, 256, 0, st>>>((T*)y, (const T*)x, (const T*)wa, (const T*)wb, (const I*)indices, \
                                                   h1, h2, rank, num_adapters, scale)
  if (dtype == TRB_F16) {
    if (index_is_64bit) TRB_LORA_IDX(__half, int64_t); else TRB_LORA_IDX(__half, int32_t);
  } else if (dtype == TRB_BF16) {
    if (index_is_64bit) TRB_LORA_IDX(__nv_bfloat16, int64_t); else TRB_LORA_IDX(__nv_bfloat16, int32_t);
  } else {
    return TRB_ERR_KERN_SHAPE;
  }
#undef TRB_LORA_IDX
  return cudaGetLastError() == cudaSuccess ? TRB_OK : TRB_ERR_CUDA;
}
