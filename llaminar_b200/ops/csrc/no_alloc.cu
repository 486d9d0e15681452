// Allocation-free C entry point of the split-K quantised GEMV (declaration and contract: no_alloc.h).
//
// The GEMV kernel needs two pieces of scratch: fp32 partial sums for the K splits and one arrival counter
// per 128-row tile.  The regular entry point takes them from buffers the Python layer allocated with torch;
// here they are a file-scope __device__ array, so nothing is allocated at run time.  In host code the name
// of a __device__ array is only a handle, not an address a kernel may dereference: the device address is
// fetched once per device with cudaGetSymbolAddress and that pointer is what the kernel receives.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>

#include "gemv.h"
#include "no_alloc.h"

namespace {

constexpr int kMaxTiles = LLAMINAR_NOALLOC_MAX_N / 128;
constexpr int kMaxDevices = 64;

struct Scratch {
    float accum[LLAMINAR_NOALLOC_MAX_ROWS * LLAMINAR_NOALLOC_MAX_N];
    unsigned tickets[kMaxTiles];
};
static __device__ __align__(256) Scratch g_scratch;

struct DeviceSlot {
    std::atomic<Scratch*> ptr{nullptr};      // published once per device; racing first callers store the same value
};
DeviceSlot g_slots[kMaxDevices];
thread_local char g_error[256] = "";

int fail(int code, const char* what, const char* detail = "") {
    std::snprintf(g_error, sizeof(g_error), "llaminar_gemv_noalloc: %s%s", what, detail);
    return code;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const char* llaminar_gemv_noalloc_error(void) { return g_error; }

extern "C" __attribute__((visibility("default"))) int llaminar_gemv_noalloc(const void* w, int fmt, int n, int k, const void* x,
                                                                            int m, void* out, void* stream) {
    g_error[0] = 0;
    if (!w || !x || !out) return fail(1, "null pointer argument");
    if (m < 1 || m > LLAMINAR_NOALLOC_MAX_ROWS) return fail(2, "m must be between 1 and 4 rows");
    if (n < 1 || k < 256 || k % 256) return fail(3, "k must be a positive multiple of 256 and n positive");
    const int n_tiles = (n + 127) / 128;
    if (n_tiles * 128 > LLAMINAR_NOALLOC_MAX_N) return fail(4, "n exceeds the built-in scratch (LLAMINAR_NOALLOC_MAX_N = 65536)");
    if (fmt < 0 || fmt > 5) return fail(5, "unknown weight format id");

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(6, "cudaGetDevice failed: ", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(7, "device index out of range");
    DeviceSlot& slot = g_slots[dev];
    Scratch* sc = slot.ptr.load(std::memory_order_acquire);
    if (!sc) {
        // one-time set-up for this device, with this device current: resolve the array's device address, and check that
        // the caller's output buffer belongs to this device (a wrong current device would otherwise pair this device's
        // scratch with another device's buffers)
        cudaPointerAttributes attr{};
        e = cudaPointerGetAttributes(&attr, out);
        if (e != cudaSuccess) return fail(11, "cudaPointerGetAttributes(out) failed: ", cudaGetErrorString(e));
        if (attr.type == cudaMemoryTypeDevice && attr.device != dev)
            return fail(12, "out belongs to another device than the current one (call cudaSetDevice first)");
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_scratch);
        if (e != cudaSuccess || !p) return fail(8, "cudaGetSymbolAddress failed: ", cudaGetErrorString(e));
        sc = static_cast<Scratch*>(p);
        slot.ptr.store(sc, std::memory_order_release);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // the array keeps whatever the previous call left: start this call's part from zero
    const size_t stride = (size_t)n_tiles * 128;
    e = cudaMemsetAsync(sc->accum, 0, (size_t)m * stride * sizeof(float), st);
    if (e == cudaSuccess) e = cudaMemsetAsync(sc->tickets, 0, (size_t)n_tiles * sizeof(unsigned), st);
    if (e != cudaSuccess) return fail(9, "clearing the scratch failed: ", cudaGetErrorString(e));

    llm::GemvParams p{};
    p.w = static_cast<const uint8_t*>(w);
    p.fmt = fmt; p.n = n; p.k = k; p.n_tiles = n_tiles; p.k_blocks = k / 256;
    p.x = x; p.x_stride = k; p.z_per_x = 1;
    p.norm_w = nullptr; p.eps = 0.f;
    p.accum = sc->accum; p.tickets = sc->tickets; p.accum_stride = (int)stride;
    p.ksplit = 0; p.epi = llm::EPI_STORE;
    p.out = out; p.out_stride = n; p.out_f32 = 0;
    p.bias = nullptr; p.expert_ids = nullptr; p.expert_stride = 0;
    e = llm::launch_gemv(p, m, 1, st);
    if (e != cudaSuccess) return fail(10, "kernel launch failed: ", cudaGetErrorString(e));
    return 0;
}
