// Thin inline-PTX wrappers shared by the tcgen05 kernels (large-tile GEMM, small-batch GEMM, prefill attention):
// mbarriers, proxy / tcgen05 fences, TMA tile loads, shared-memory and instruction descriptors, MMA issue / commit and
// TMEM loads.  Policy (how long a wait may spin, what happens on a timeout) stays with each kernel.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace llm {
namespace tc5 {

LLM_DEVICE void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
LLM_DEVICE void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
LLM_DEVICE void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
LLM_DEVICE unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
LLM_DEVICE bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// One lane of a converged warp, chosen by the hardware.  A single-lane region entered through elect.sync keeps its operands
// in uniform registers; the same region behind `if (lane == 0)` issued tcgen05.mma at 53-140 clocks apiece (measured, one
// warp, M=128 N=32 K=16), behind elect.sync at 16 clocks, which is the tensor pipe's own rate for that shape.
LLM_DEVICE bool elect_one() {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok));
    return ok != 0;
}
// ---- bounded mbarrier waits shared by the tcgen05 kernels ----
constexpr unsigned long long WAIT_LIMIT_NS = 2000ull * 1000 * 1000;     // 2 s: far beyond any wait inside one launch, and beyond a host hiccup of a peer rank
#ifndef LLM_WAIT_HINT_NS
#define LLM_WAIT_HINT_NS 4000
#endif
constexpr uint32_t WAIT_HINT_NS = LLM_WAIT_HINT_NS;       // suspend-time hint of one try_wait
constexpr uint32_t WAIT_TRIES = 32;           // attempts inside one assembly loop, between two looks at the abort flag and the clock
// `tries` attempts of mbarrier.try_wait in one assembly block.  The loop is invisible to the compiler, so it plants no
// divergence bookkeeping around it; try_wait answers a whole warp at once, so the lanes leave together anyway.
LLM_DEVICE uint32_t mbar_try_wait_loop(uint32_t bar, uint32_t parity, uint32_t tries) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .u32 n;\n\tmov.u32 n, %3;\n"
        "WAIT_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %4;\n\t"
        "@p bra WAIT_DONE;\n\t"
        "sub.u32 n, n, 1;\n\t"
        "setp.ne.u32 p, n, 0;\n\t"
        "@p bra WAIT_LOOP;\n"
        "WAIT_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(tries), "r"(WAIT_HINT_NS) : "memory");
    return ok;
}
// Bounded wait.  abort_flag[0]: some wait of this CTA gave up (everybody leaves).  abort_flag[1]: the epilogue is inside its
// own bounded wait for a tensor-parallel peer; the pipeline behind it is legitimately stalled, so the clock is restarted
// meanwhile (the peer wait has its own limit and reports through the status word).
// WARP = true: called by all 32 lanes of a converged warp; the result is made warp-uniform by a vote, so the branches on it
// are uniform branches.  WARP = false: called by a single elected lane.
template <bool WARP>
LLM_DEVICE bool mbar_wait_t(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    uint32_t ok = mbar_try_wait_loop(bar, parity, WAIT_TRIES);
    if (WARP) ok = __all_sync(0xffffffffu, ok);
    if (ok) return true;
    unsigned long long t0 = 0;
#pragma unroll 1
    for (;;) {
        int give_up = abort_flag[0];
        const unsigned long long now = global_timer_ns();
        if (t0 == 0 || abort_flag[1]) t0 = now;
        else if (now - t0 > WAIT_LIMIT_NS) give_up = 1;
        if (WARP) give_up = __any_sync(0xffffffffu, give_up);
        if (give_up) break;
        ok = mbar_try_wait_loop(bar, parity, WAIT_TRIES);
        if (WARP) ok = __all_sync(0xffffffffu, ok);
        if (ok) return true;
    }
    abort_flag[0] = 1;
    return false;
}
LLM_DEVICE bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) { return mbar_wait_t<false>(bar, parity, abort_flag); }
LLM_DEVICE bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) { return mbar_wait_t<true>(bar, parity, abort_flag); }
// arrive from the lanes whose `pred` is set, without a branch the compiler would have to reconverge
LLM_DEVICE void mbar_arrive_if(uint32_t bar, bool pred) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %1, 0;\n\t@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}" ::"r"(bar), "r"((uint32_t)pred) : "memory");
}
LLM_DEVICE void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
LLM_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
LLM_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// untiled bulk copy global -> this CTA's shared memory; both addresses 16-byte aligned, size a multiple of 16 bytes
LLM_DEVICE void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// one tile of a 2-D tensor map into shared memory (no multicast: the tile is for this CTA only)
LLM_DEVICE void tma_load_2d(uint32_t dst, const CUtensorMap* tmap, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(bar) : "memory");
}

// K-major, 128-byte swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
LLM_DEVICE uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fff);          // start address
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                          // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
    return d;
}
// bf16 x bf16 -> fp32, both operands K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// A and B from shared memory
LLM_DEVICE void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// A from tensor memory, B from shared memory
LLM_DEVICE void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
LLM_DEVICE void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 accumulator columns of this warp's 32 TMEM lanes; the values may be read only after tmem_wait_ld on the same array
LLM_DEVICE void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
// Completes every tcgen05.ld of this thread; the empty statements tie the array to the wait so that no use of it is scheduled earlier.
LLM_DEVICE void tmem_wait_ld(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) asm volatile("" : "+r"(r[i]));
}

LLM_DEVICE unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
LLM_DEVICE void red_release_gpu_add(unsigned* p, unsigned v) { asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

}  // namespace tc5
}  // namespace llm
