// trb_sbmm_indexed_static: the fused indexed delta matmul for callers that have no way to give
// the library a scratch buffer.
//
// trb_sbmm_indexed needs working memory (router counters, the sorted-token permutation, the tile
// list and the gathered activation rows) and expects the caller to allocate it.  Some hosts cannot:
// a serving process that handed all of HBM to its own arena at start-up and has no allocator
// hook for foreign code, or a plugin slot whose contract forbids cudaMalloc once initialisation is
// over because the call stalls every stream of the device.  For them the working memory is a
// fixed array that is part of the library image itself.
#pragma once

#include <mutex>

#include "common.cuh"

// Limit: what trb_sbmm_indexed_scratch_min_bytes(T, K, D) reports must fit in this array
// (e.g. T <= 256 tokens with K <= 8192, or T <= 512 with K <= 4096).  Every GPU that loads the
// library carries the array from the first use of the library on it until the process exits.
#define TRB_STATIC_SCRATCH_BYTES (4u * 1024u * 1024u + 64u * 1024u)

namespace trb {

static __device__ __align__(256) unsigned char g_static_scratch[TRB_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, never a device address: the
// address a kernel may use comes from cudaGetSymbolAddress, asked once per device while that
// device is current.
static int static_scratch_address(int dev, void** out) {
  static std::mutex mu;
  static void* addr[64] = {};
  static bool known[64] = {};
  if (dev < 0 || dev >= 64) return TRB_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(mu);
  if (!known[dev]) {
    if (cudaSetDevice(dev) != cudaSuccess) return TRB_ERR_CUDA;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return TRB_ERR_CUDA;
    addr[dev] = p;
    known[dev] = true;
  }
  *out = addr[dev];
  return TRB_OK;
}

}  // namespace trb

extern "C" size_t trb_sbmm_indexed_static_capacity(void) { return TRB_STATIC_SCRATCH_BYTES; }

extern "C" int trb_sbmm_indexed_static(const void* x, const void* qweights, const void* metas, const void* scales,
                                       const void* indices, void* y, int num_tokens, int prob_m, int prob_k,
                                       int num_deltas, int index_offset, int groupsize, int accumulate, int dev,
                                       void* stream) {
  using namespace trb;
  if (num_tokens < 0 || prob_k < 0 || num_deltas <= 0) return TRB_ERR_BAD_ARG;
  // Sizes beyond the array are refused before anything is launched.
  if (trb_sbmm_indexed_scratch_min_bytes(num_tokens, prob_k, num_deltas) > (size_t)TRB_STATIC_SCRATCH_BYTES)
    return TRB_ERR_SCRATCH;
  void* scratch = nullptr;
  const int rc = static_scratch_address(dev, &scratch);
  if (rc != TRB_OK) return rc;
  // Nothing in the array has to start at zero: the router rewrites the counters, the permutation
  // and the tile list on every call, the gather kernel zeroes the K-split counters, and the
  // grouped kernel reads only the rows the tile list names.
  return trb_sbmm_indexed(x, qweights, metas, scales, indices, y, num_tokens, prob_m, prob_k, num_deltas,
                          index_offset, groupsize, accumulate, scratch, TRB_STATIC_SCRATCH_BYTES, dev, stream);
}
