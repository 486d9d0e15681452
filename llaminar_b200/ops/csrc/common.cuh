// Shared device helpers for the sm_100a kernels of this extension.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLM_DEVICE __device__ __forceinline__

namespace llm {

constexpr int TILE_N = 128;   // rows per weight chunk
constexpr int TILE_K = 256;   // columns per weight chunk

// Status codes a kernel may leave in a caller-provided status word (never traps).
enum KernelStatus : int { STATUS_OK = 0, STATUS_TIMEOUT = 1, STATUS_BAD_ARG = 2, STATUS_BAD_INDEX = 3 };

// Debug build with explicit bounds checks (-DLLM_BOUNDS_CHECK; `LLAMINAR_BOUNDS_CHECK=1` builds it into its own directory).
// Every index that a kernel takes from a device-side table (KV page ids, block-table rows) goes through LLM_CHECK_INDEX:
// an index outside [0, hi) raises STATUS_BAD_INDEX in the translation unit's status word and is replaced by 0, so the
// access stays inside the allocation and the host reads the word (`ops.bounds_status()`) instead of the GPU faulting.
// The production build compiles the macro away.
#ifdef LLM_BOUNDS_CHECK
static __device__ int g_bounds_status;
__device__ __forceinline__ bool llm_index_in_range(long long v, long long hi) {
    const bool ok = v >= 0 && v < hi;
    if (!ok) atomicExch(&g_bounds_status, (int)STATUS_BAD_INDEX);
    return ok;
}
#define LLM_CHECK_INDEX(v, hi) (llm::llm_index_in_range((long long)(v), (long long)(hi)) ? (v) : 0)
#define LLM_DEFINE_BOUNDS_STATUS_READER(fn)                                              \
    int fn(bool reset) {                                                                 \
        int v = 0;                                                                       \
        cudaMemcpyFromSymbol(&v, g_bounds_status, sizeof(int));                          \
        if (reset && v) { const int z = 0; cudaMemcpyToSymbol(g_bounds_status, &z, sizeof(int)); } \
        return v;                                                                        \
    }
#else
#define LLM_CHECK_INDEX(v, hi) (v)
#define LLM_DEFINE_BOUNDS_STATUS_READER(fn) \
    int fn(bool) { return 0; }
#endif

LLM_DEVICE float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
LLM_DEVICE float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

LLM_DEVICE float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
LLM_DEVICE float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
LLM_DEVICE uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
LLM_DEVICE float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

LLM_DEVICE uint4 ldg_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
LLM_DEVICE uint2 ldg_nc_v2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
LLM_DEVICE uint32_t ldg_nc_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
LLM_DEVICE uint16_t ldg_nc_u16(const void* p) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// Programmatic dependent launch (see launch.h): trigger lets the next kernel of the stream start its prologue, wait blocks
// until the previous kernel has completed and its memory is visible.  Both are no-ops for an ordinary launch.
// A kernel launched that way becomes resident while its predecessor still runs, so whatever
// the predecessor writes is NOT read-only for this kernel's lifetime: after `pdl_wait()` read it with ordinary or `__ldcg`
// loads, never through the read-only path (`ld.global.nc`, `__ldg`, or a `const __restrict__` parameter, which lets the
// compiler pick that path).  A line that another CTA on the same SM brought into the read-only cache while the predecessor had
// not yet written it would be served stale.  Weights and other constants may use it.
LLM_DEVICE void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
LLM_DEVICE void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

LLM_DEVICE uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// branch-free: the approximate division has no slow path for huge or infinite denominators (they give 0, the right limit)
LLM_DEVICE float silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

}  // namespace llm
