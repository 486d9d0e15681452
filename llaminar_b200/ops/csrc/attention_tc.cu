// Paged causal GQA prefill attention on the 5th-generation tensor cores (head_dim 128).
//
// One CTA = 128 query rows of one head.  Keys are walked in tiles of 128 (two 64-token pages):
//   S = Q K^T          tcgen05.mma, M = 128 query rows, N = 128 keys, K = head_dim, fp32 accumulator in TMEM (two buffers)
//   softmax            two threads per query row (== TMEM lane), 64 columns each: tcgen05.ld, running max / sum in registers,
//                      P = exp2(...) written as bf16 into a swizzled shared-memory operand tile
//   O_tile = P V       tcgen05.mma, M = 128 query rows, N = head_dim, K = 128 keys, accumulator in TMEM; the softmax
//                      threads read it back and fold it into their register copy of the output row (scaled by the
//                      running-max correction), so no accumulator in TMEM ever needs rescaling.
// Every MMA operand is a K-major, 128-byte-swizzled shared-memory tile.  K pages have that form already (a key row is
// head_dim contiguous values); V is needed as V^T (head_dim rows x keys), so the loader warps stage a page with cp.async
// and transpose it 8x8 block by block with ldmatrix.trans + stmatrix.  Q, K and V^T are written by ordinary stores /
// cp.async and handed to the tensor core after fence.proxy.async.
//
// Roles (384 threads): warps 0-7 softmax + output (warps w and w + 4 share 32 query rows and take 64 columns each),
// warps 8-10 loaders, warp 11 TMEM allocation + MMA issue.
// Every mbarrier wait is bounded; on a timeout the kernel raises the status word and tears down cleanly.
//
// Replaces flash_attention_2_pipelined_kernel of the reference (src/v2/kernels/cuda/attention/CUDAFlashAttentionKernels.cu:348).
#include "ops.h"
#include "tc_common.cuh"

namespace llm {
namespace atc {
using namespace tc5;

constexpr int D = 128, BQ = 128, BK = 128, PAGE = 64;
constexpr int ATOM = 128 * 128;                    // 128 rows x 64 bf16: one swizzled operand atom
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int THREADS = 384, N_LOADERS = 96;            // 8 softmax warps, 3 loader warps, 1 MMA warp

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr int OFF_Q = 0;                           // 2 atoms (d halves)
constexpr int OFF_K = OFF_Q + 2 * ATOM;            // 2 buffers x 2 atoms (d halves)
constexpr int OFF_VT = OFF_K + 4 * ATOM;           // 2 buffers x 2 atoms (key halves), rows = d
constexpr int OFF_P = OFF_VT + 4 * ATOM;           // 2 atoms (key halves), rows = q
constexpr int OFF_VS = OFF_P + 2 * ATOM;           // staging of the two V pages of a key tile: 128 keys x 256 bytes
constexpr int SMEM_BYTES = OFF_VS + BK * D * 2 + 1024;

LLM_DEVICE void cp_async16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
LLM_DEVICE void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
LLM_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
LLM_DEVICE void cp_async_wait_1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// bf16 x bf16 -> fp32, both operands K-major, M = 128, N = 128
constexpr uint32_t IDESC = instr_desc(128);
LLM_DEVICE float ex2(float x) {                    // 2^x, approximate; -inf -> 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 16-byte unit `unit` (0..7) of row `row` inside one operand atom
LLM_DEVICE uint32_t atom_addr(uint32_t atom_base, int row, int unit) { return atom_base + row * 128 + (((unit ^ row) & 7) << 4); }
// staging tile of a V page: rows of 256 bytes, 16-byte units XOR-swizzled inside groups of eight
LLM_DEVICE uint32_t stage_addr(uint32_t base, int row, int unit) { return base + row * 256 + (((unit & ~7) | ((unit ^ row) & 7)) << 4); }

LLM_DEVICE void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
LLM_DEVICE void stmatrix_x4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}

enum Bar { K_FULL = 0, K_EMPTY = 2, VT_FULL = 4, VT_EMPTY = 6, S_FULL = 8, S_EMPTY = 10, P_FULL = 12, O_FULL = 13, O_EMPTY = 14, LD_SYNC = 15, PAIR = 16, N_BARS = 20 };

__global__ void __launch_bounds__(THREADS, 1) paged_attn_prefill_tc_kernel(const AttnPrefillParams p, int* status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_bars[N_BARS];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort[2];       // [1] stays 0 here (tc_common.cuh: restarts the wait clock when set)
    // [column half][row]: row maxima (and, at the end, sums) of a thread pair.  One copy is enough: a thread overwrites its
    // entry only after the O_FULL wait of the tile, which needs the partner's P_FULL arrival, which follows the partner's read.
    __shared__ float s_xchg[2][BQ];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head = blockIdx.y, seq = blockIdx.z;
    const int G = p.n_heads / p.n_kv_heads, kvh = head / G;
    const int q_start = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_start;
    // the last query tiles see the most keys: they go first so that the grid ends with the short CTAs
    const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BQ;
    if (q0 >= q_len) return;                               // uniform for the CTA, before any barrier or allocation
    const int ctx = p.ctx_lens[seq];                       // tokens already in the cache before this chunk
    const int rows = min(BQ, q_len - q0);
    const int kv_end = ctx + q0 + rows;                    // keys this query tile can see
    const int nt = (kv_end + BK - 1) / BK, n_pages = (kv_end + PAGE - 1) / PAGE;
    const int* btab = p.block_table + (size_t)seq * p.max_pages;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base + OFF_Q, sK = base + OFF_K, sVT = base + OFF_VT, sP = base + OFF_P, sVS = base + OFF_VS;
    const uint32_t bars = smem_u32(s_bars);
    auto bar = [&](int i) { return bars + i * 8; };

    if (tid == 0) {
        s_abort[0] = 0; s_abort[1] = 0;
        const int counts[N_BARS] = {3, 3, 1, 1, 3, 3, 1, 1, 1, 1, 8, 8, 8, 1, 8, 3, 2, 2, 2, 2};
        for (int i = 0; i < N_BARS; ++i) mbar_init(bar(i), counts[i]);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 11) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    volatile int* abort_flag = s_abort;

    if (warp < 8) {
        // ------------------------------ softmax + output: two threads per query row (== TMEM lane), 64 columns each ------------------------------
        // (one warp per scheduler converting whole rows needed ~4.4 us per key tile; halving the row doubles the warps per
        // scheduler and halves the work of each)
        const int row = tid & 127, half = tid >> 7, q4 = warp & 3;
        const bool valid = row < rows;
        const int lim = ctx + min(q0 + row, q_len - 1) + 1;           // this row sees keys < lim
        const uint32_t t_lane = tmem + ((uint32_t)(q4 * 32) << 16) + half * 64;
        const float sl2 = p.scale * 1.4426950408889634f;
        constexpr int HD = D / 2;
        float o[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] = 0.f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        int n_pair = 0;
        auto pair_meet = [&]() {                   // bounded rendezvous of the two warps that share these 32 rows
            __syncwarp();
            mbar_arrive_if(bar(PAIR + q4), lane == 0);
            const bool r = mbar_wait_warp(bar(PAIR + q4), n_pair & 1, abort_flag);
            ++n_pair;
            return r;
        };
        uint32_t ra[32], rb[32];
        float m_new = -INFINITY, mb = 0.f, alpha = 0.f, alpha_prev = 0.f;
        // first pass over tile j: wait for S, row maximum over this thread's 64 columns, exchange with the partner thread
        auto pass1 = [&](int j) {
            const int b = j & 1;
            if (!mbar_wait_warp(bar(S_FULL + b), (j >> 1) & 1, abort_flag)) return false;
            tc_fence_after();
            const int key0 = j * BK + half * 64;
            const uint32_t t_s = t_lane + b * 128;
            tmem_ld32_issue(t_s, ra);
            tmem_ld32_issue(t_s + 32, rb);
            tmem_wait_ld(ra);
            tmem_wait_ld(rb);
            float mx = -INFINITY;
            if (key0 + 64 > lim) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float s0 = key0 + i >= lim ? -INFINITY : __uint_as_float(ra[i]);
                    const float s1 = key0 + 32 + i >= lim ? -INFINITY : __uint_as_float(rb[i]);
                    mx = fmaxf(mx, fmaxf(s0, s1));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(ra[i]), __uint_as_float(rb[i])));
            }
            s_xchg[half][row] = mx;
            if (!pair_meet()) return false;
            mx = fmaxf(mx, s_xchg[half ^ 1][row]);
            m_new = fmaxf(m, mx * sl2);
            mb = m_new == -INFINITY ? 0.f : m_new;
            alpha = ex2(m - mb);
            return true;
        };
        // the tile's P V product is complete: fold it into the register copy of the output row
        auto fold = [&](int j) {
            if (!mbar_wait_warp(bar(O_FULL), j & 1, abort_flag)) return false;
            tc_fence_after();
            const uint32_t t_o = t_lane + 256;
            tmem_ld32_issue(t_o, ra);
            tmem_ld32_issue(t_o + 32, rb);
            tmem_wait_ld(ra);
            tmem_wait_ld(rb);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                o[i] = o[i] * alpha_prev + __uint_as_float(ra[i]);
                o[32 + i] = o[32 + i] * alpha_prev + __uint_as_float(rb[i]);
            }
            tc_fence_before();
            __syncwarp();
            mbar_arrive_if(bar(O_EMPTY), lane == 0);
            return true;
        };
        // Order per tile: first pass (row maxima; the P V MMAs of the previous tile run meanwhile) -> fold of the previous tile
        // (which also frees the P tile) -> second pass (P).  Every phase has exactly one call site: the unrolled 64-column
        // loops are large and a second copy of each showed up as instruction-fetch stalls.
        for (int j = 0; j <= nt && ok; ++j) {
            const int b = j & 1;
            if (j < nt) ok = pass1(j);
            if (ok && j > 0) ok = fold(j - 1);
            if (!ok || j == nt) break;
            const int key0 = j * BK + half * 64;
            const bool need_mask = key0 + 64 > lim;
            const uint32_t t_s = t_lane + b * 128;
            tmem_ld32_issue(t_s, ra);
            tmem_ld32_issue(t_s + 32, rb);
            tmem_wait_ld(ra);
            tmem_wait_ld(rb);
            float sum = 0.f;
            auto probs_of = [&](int c, const uint32_t (&r)[32]) {
                uint32_t w[16];
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const int key = key0 + c * 32 + i;
                        const float p0 = key >= lim ? 0.f : ex2(__uint_as_float(r[i]) * sl2 - mb);
                        const float p1 = key + 1 >= lim ? 0.f : ex2(__uint_as_float(r[i + 1]) * sl2 - mb);
                        sum += p0 + p1;
                        w[i >> 1] = pack_bf16(p0, p1);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = ex2(__uint_as_float(r[i]) * sl2 - mb), p1 = ex2(__uint_as_float(r[i + 1]) * sl2 - mb);
                        sum += p0 + p1;
                        w[i >> 1] = pack_bf16(p0, p1);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t dst = atom_addr(sP + half * ATOM, row, c * 4 + u);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(w[4 * u]), "r"(w[4 * u + 1]), "r"(w[4 * u + 2]), "r"(w[4 * u + 3]) : "memory");
                }
            };
            probs_of(0, ra);
            probs_of(1, rb);
            tc_fence_before();
            fence_proxy_async();
            __syncwarp();
            mbar_arrive_if(bar(S_EMPTY + b), lane == 0); mbar_arrive_if(bar(P_FULL), lane == 0);
            l = l * alpha + sum;
            m = m_new;
            alpha_prev = alpha;
        }
        // the row's normaliser is the sum over both column halves
        if (ok) {
            s_xchg[half][row] = l;
            ok = pair_meet();
        }
        if (ok && valid) {
            const float lt = l + s_xchg[half ^ 1][row];
            const float inv = lt > 0.f ? 1.f / lt : 0.f;
            __nv_bfloat16* dst = p.out + ((size_t)(q_start + q0 + row) * p.n_heads + head) * D + half * HD;
#pragma unroll
            for (int u = 0; u < HD / 8; ++u) {
                uint4 v;
                v.x = pack_bf16(o[8 * u] * inv, o[8 * u + 1] * inv); v.y = pack_bf16(o[8 * u + 2] * inv, o[8 * u + 3] * inv);
                v.z = pack_bf16(o[8 * u + 4] * inv, o[8 * u + 5] * inv); v.w = pack_bf16(o[8 * u + 6] * inv, o[8 * u + 7] * inv);
                *reinterpret_cast<uint4*>(dst + 8 * u) = v;
            }
        }
    } else if (warp < 11) {
        // ------------------------------ loaders: Q once, then K and V^T of every key tile ------------------------------
        const int lt = tid - 256, lw = warp - 8;
        for (int idx = lt; idx < BQ * 16; idx += N_LOADERS) {
            const int r = idx >> 4, u = idx & 15;
            const uint32_t dst = atom_addr(sQ + (u >> 3) * ATOM, r, u & 7);
            if (r < rows) cp_async16(dst, p.q + ((size_t)(q_start + q0 + r) * p.n_heads + head) * D + u * 8);
            else asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0u) : "memory");
        }
        int n_sync = 0;
        bool ok = true;
        auto loaders_meet = [&]() {               // bounded rendezvous of the loader warps
            __syncwarp();
            mbar_arrive_if(bar(LD_SYNC), lane == 0);
            const bool r = mbar_wait_warp(bar(LD_SYNC), n_sync & 1, abort_flag);
            ++n_sync;
            return r;
        };
        // a page past the end repeats the last one (its keys are masked)
        auto page_of = [&](int pg) { return (size_t)LLM_CHECK_INDEX(btab[min(pg, n_pages - 1)], p.n_pages); };
        auto issue_k = [&](int j) {                // K tile j -> operand buffer j & 1 (one cp.async group, also when j >= nt)
            if (j < nt) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const __nv_bfloat16* kp = p.kv + ((page_of(2 * j + half) * 2 + 0) * p.n_kv_heads + kvh) * (size_t)(PAGE * D);
                    for (int idx = lt; idx < PAGE * 16; idx += N_LOADERS) {
                        const int r = idx >> 4, u = idx & 15;
                        cp_async16(atom_addr(sK + ((j & 1) * 2 + (u >> 3)) * ATOM, half * PAGE + r, u & 7), kp + r * D + u * 8);
                    }
                }
            }
            cp_async_commit();
        };
        auto issue_v = [&](int j) {                // the two V pages of tile j -> staging (one cp.async group)
            if (j < nt) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const __nv_bfloat16* vp = p.kv + ((page_of(2 * j + half) * 2 + 1) * p.n_kv_heads + kvh) * (size_t)(PAGE * D);
                    for (int idx = lt; idx < PAGE * 16; idx += N_LOADERS) {
                        const int r = idx >> 4, u = idx & 15;
                        cp_async16(stage_addr(sVS, half * PAGE + r, u), vp + r * D + u * 8);
                    }
                }
            }
            cp_async_commit();
        };
        // Copies run one tile ahead: K of tile j + 1 is in flight while V of tile j is transposed, V of tile j + 1 while the
        // loaders wait for the next K buffer.  Groups are committed in the order K0 (with Q), V0, K1, V1, ...
        issue_k(0);
        issue_v(0);
        for (int j = 0; j < nt && ok; ++j) {
            const int b = j & 1;
            cp_async_wait_1();                     // K of tile j (and Q) has landed; V of tile j may still be in flight
            fence_proxy_async();
            __syncwarp();
            mbar_arrive_if(bar(K_FULL + b), lane == 0);
            if (j + 1 < nt) ok = mbar_wait_warp(bar(K_EMPTY + (b ^ 1)), (((j + 1) >> 1) & 1) ^ 1, abort_flag);
            if (!ok) break;
            issue_k(j + 1);
            cp_async_wait_1();                     // V of tile j has landed (K of tile j + 1 may still be in flight)
            ok = mbar_wait_warp(bar(VT_EMPTY + b), ((j >> 1) & 1) ^ 1, abort_flag) && loaders_meet();
            if (!ok) break;
            // transpose 8x8 blocks: 16 key blocks x 4 groups of four d blocks
            for (int op = lw; op < 64; op += N_LOADERS / 32) {
                const int kb = op >> 2, dg = op & 3, mi = lane >> 3, r = lane & 7;
                uint32_t r0, r1, r2, r3;
                ldmatrix_x4_trans(stage_addr(sVS, kb * 8 + r, dg * 4 + mi), r0, r1, r2, r3);
                stmatrix_x4(atom_addr(sVT + (b * 2 + (kb >> 3)) * ATOM, dg * 32 + mi * 8 + r, kb & 7), r0, r1, r2, r3);
            }
            fence_proxy_async();
            ok = loaders_meet();                   // the staging tile may be overwritten
            if (!ok) break;
            mbar_arrive_if(bar(VT_FULL + b), lane == 0);
            issue_v(j + 1);
        }
        cp_async_wait_all();
    } else if (elect_one()) {
        // ------------------------------ MMA issue ------------------------------
        bool ok = true;
        auto issue_s = [&](int j) {
            const int b = j & 1;
            ok = mbar_wait(bar(K_FULL + b), (j >> 1) & 1, abort_flag) && mbar_wait(bar(S_EMPTY + b), ((j >> 1) & 1) ^ 1, abort_flag);
            if (!ok) return;
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                mma_f16(tmem + b * 128, smem_desc_sw128(sQ + (ks >> 2) * ATOM) + 2 * (ks & 3),
                        smem_desc_sw128(sK + (b * 2 + (ks >> 2)) * ATOM) + 2 * (ks & 3), IDESC, ks > 0 ? 1u : 0u);
            mma_commit(bar(S_FULL + b));
            mma_commit(bar(K_EMPTY + b));
        };
        issue_s(0);
        for (int j = 0; j < nt && ok; ++j) {
            const int b = j & 1;
            if (j + 1 < nt) issue_s(j + 1);
            if (!ok) break;
            ok = mbar_wait(bar(P_FULL), j & 1, abort_flag) && mbar_wait(bar(VT_FULL + b), (j >> 1) & 1, abort_flag) &&
                 mbar_wait(bar(O_EMPTY), (j & 1) ^ 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                mma_f16(tmem + 256, smem_desc_sw128(sP + (ks >> 2) * ATOM) + 2 * (ks & 3),
                        smem_desc_sw128(sVT + (b * 2 + (ks >> 2)) * ATOM) + 2 * (ks & 3), IDESC, ks > 0 ? 1u : 0u);
            mma_commit(bar(O_FULL));
            mma_commit(bar(VT_EMPTY + b));
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    if (s_abort[0]) {
        if (tid == 0 && status) atomicExch(status, (int)STATUS_TIMEOUT);
        for (int i = 0; i < 2000; ++i) __nanosleep(100);      // let copies still in flight land before the memory is reused
        __syncthreads();
    }
    if (warp == 11) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}

}  // namespace atc

cudaError_t launch_attn_prefill_tc(const AttnPrefillParams& p, int n_seqs, int max_q_len, int* status, cudaStream_t st) {
    if (n_seqs == 0 || max_q_len == 0) return cudaSuccess;
    if (p.head_dim != atc::D || p.n_heads % p.n_kv_heads) return cudaErrorInvalidValue;
    static bool once = false;
    if (!once) {
        cudaError_t e = cudaFuncSetAttribute(atc::paged_attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, atc::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        once = true;
    }
    dim3 grid((max_q_len + atc::BQ - 1) / atc::BQ, p.n_heads, n_seqs);
    atc::paged_attn_prefill_tc_kernel<<<grid, atc::THREADS, atc::SMEM_BYTES, st>>>(p, status);
    return cudaGetLastError();
}

LLM_DEFINE_BOUNDS_STATUS_READER(bounds_status_attention_tc)

}  // namespace llm
