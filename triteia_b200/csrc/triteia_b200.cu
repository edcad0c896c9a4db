// The library is built as ONE translation unit (no relocatable device code): every kernel and
// every extern "C" entry point declared in include/triteia_b200.h is reached from here.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "route.cuh"
#include "delta_gemm.cuh"
#include "tc_common.cuh"
#include "delta_gemm_tcsp.cuh"
#include "delta_gemm_host.cuh"
#include "shard.cuh"
#include "unpack.cuh"
#include "pack.cuh"
#include "stack.cuh"
#include "lora.cuh"
#include "base_gemm.cuh"
#include "elementwise.cuh"
#include "no_alloc.cuh"
