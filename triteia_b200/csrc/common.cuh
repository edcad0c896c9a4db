// Device-side building blocks shared by the kernels: mbarrier pipeline primitives with
// bounded waits, TMA (cp.async.bulk.tensor) loads, ldmatrix, the 2:4-sparse MMA and the
// int4 -> fp16 conversion.  sm_100a only.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/triteia_b200.h"

namespace trb {

// ---------------------------------------------------------------------------------------------
// Device error word.  A kernel that gives up on a bounded wait records it here; the host reads
// it through trb_device_status().
// ---------------------------------------------------------------------------------------------
__device__ int g_device_status = 0;  // the library is one translation unit

// Upper bound on polls of one mbarrier wait.  Each poll is a try_wait that itself suspends for
// a hardware-defined interval, so this is tens of milliseconds at the very least.
constexpr uint32_t kMaxPolls = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                   smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
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

// Shared-memory loads through a 32-bit shared address: constant offsets fold into the instruction.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// Bounded wait.  `dead` is a CTA-wide shared flag: once any wait of the CTA has expired every
// later wait returns at once, so a broken pipeline drains in bounded time instead of hanging.
// The launch's output is then garbage and g_device_status says so.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* dead,
                                          uint32_t max_polls = kMaxPolls) {
  if (mbar_try_wait(bar, parity)) return;
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return;
    if ((polls & 15u) == 0 && *dead) return;   // the flag is a shared-memory read: not on every poll
    if (++polls > max_polls) {
      *dead = 1;
      atomicExch(&g_device_status, TRB_ERR_TIMEOUT);
      return;
    }
  }
}

// 2-D tiled TMA load, completion signalled on an mbarrier as transaction bytes.
// c0 is the innermost coordinate (elements); c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, int c0, int c1,
                                                 uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Four 8x8 b16 matrices; lane l supplies the row address of matrix l / 8, row l % 8.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
}

// D[16x8] += A_sparse[16x32 dense, 16x16 stored] * B[32x8]; fp16 inputs, fp32 accumulate.
// a0..a3: stored A fragment (m16n8k16 A layout); e: 2:4 metadata word; SEL: which thread pair
// of each quad supplies the metadata.
template <int SEL>
__device__ __forceinline__ void mma_sp_m16n8k32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, const uint32_t (&b)[4], uint32_t e) {
  asm(
      "mma.sp::ordered_metadata.sync.aligned.m16n8k32.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9,%10,%11}, {%0,%1,%2,%3}, %12, %13;"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(e),
        "n"(SEL));
}

// Same with a zero accumulator input: D = A_sparse * B.
template <int SEL>
__device__ __forceinline__ void mma_sp_m16n8k32_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                     uint32_t a3, const uint32_t (&b)[4], uint32_t e) {
  asm(
      "mma.sp::ordered_metadata.sync.aligned.m16n8k32.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9,%10,%11}, {%12,%12,%12,%12}, %13, %14;"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "f"(0.f), "r"(e),
        "n"(SEL));
}

__device__ __forceinline__ void named_bar_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Dense m16n8k16 fp16 MMA (LoRA kernels).
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_m16n8k16_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                  uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int LUT>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(r) : "r"(a), "r"(b), "r"(c), "n"(LUT));
  return r;
}

// Nibbles 0 and 4 of q -> lo (two exact fp16 levels, code - 8), nibbles 1 and 5 -> hi.
// Uses the 0x6400 exponent trick: (0x6400 | c) is 1024 + c as fp16; nibbles taken in place at
// bit 4 carry a factor 16 that the fma removes.
__device__ __forceinline__ void int4x4_to_half2x2(uint32_t q, uint32_t& lo, uint32_t& hi) {
  constexpr uint32_t kLo = 0x000f000f, kHi = 0x00f000f0, kEx = 0x64006400;
  uint32_t l = lop3<(0xf0 & 0xcc) | 0xaa>(q, kLo, kEx);
  uint32_t h = lop3<(0xf0 & 0xcc) | 0xaa>(q, kHi, kEx);
  const uint32_t kSub = 0x64086408;  // 1032 = 1024 + 8
  const uint32_t kMul = 0x2c002c00;  // 1/16
  const uint32_t kAdd = 0xd480d480;  // -72: (1024 + 16 c) / 16 - 72 = c - 8
  __half2 lr = __hsub2(*reinterpret_cast<__half2*>(&l), *reinterpret_cast<const __half2*>(&kSub));
  __half2 hr = __hfma2(*reinterpret_cast<__half2*>(&h), *reinterpret_cast<const __half2*>(&kMul),
                       *reinterpret_cast<const __half2*>(&kAdd));
  lo = *reinterpret_cast<uint32_t*>(&lr);
  hi = *reinterpret_cast<uint32_t*>(&hr);
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while its predecessor in the stream still runs; pdl_wait() returns once that predecessor has
// completed and its writes are visible (no-op without the attribute).  pdl_launch_dependents() lets
// the successor start early (no-op when the successor was launched without the attribute).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t s) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&s));
  return *reinterpret_cast<uint32_t*>(&r);
}

}  // namespace trb
