// Paged causal GQA attention over a bf16 KV cache.
//
//   paged_attn_decode   few query rows per sequence (1 for plain decode, up to 4 for speculative
//                       verify).  The GQA group x rows are packed into the 16-row M dimension of the
//                       MMA, each warp streams its own 16 keys of every 64-token page through a private
//                       cp.async ring (no block barriers in the main loop), the sequence is split over
//                       blockIdx.y and the last CTA of a (sequence, kv head) merges the split partials.
//   paged_attn_prefill  64 query rows per CTA (16 per warp), K/V pages double-buffered for the CTA.
//
// KV cache layout (one tensor per layer): [n_pages][2 (K,V)][n_kv_heads][64 tokens][head_dim] bf16.
// Inside shared memory every 16-byte unit of a key row is XOR-swizzled with (row & 7) so ldmatrix
// is bank-conflict free.
//
// Replaces flash_attention_2_pipelined_kernel / flash_decoding_*_kernel (+ reduce) of the reference
// (reference: src/v2/kernels/cuda/attention/CUDAFlashAttentionKernels.cu:348, :923-1181).
#include "common.cuh"
#include "launch.h"
#include "ops.h"

namespace llm {

constexpr int PAGE = 64;

LLM_DEVICE void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
LLM_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> LLM_DEVICE void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

LLM_DEVICE void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
LLM_DEVICE void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
LLM_DEVICE void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

LLM_DEVICE void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool F16> LLM_DEVICE void mma_16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (F16) mma_f16(c, a, b0, b1); else mma_bf16(c, a, b0, b1);
}
LLM_DEVICE uint32_t pack_f16(float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// One 16-key x D sub-tile of K or V: row stride D*2 bytes, 16-byte units swizzled by (row & 7).
template <int D>
LLM_DEVICE uint32_t tile_addr(uint32_t base, int row, int unit) {
    return base + row * (D * 2) + (((unit & ~7) | ((unit ^ row) & 7)) << 4);
}

// S(16 x 16 keys) = Q(16 x D) K^T for one warp;  qa: the warp's Q fragments, kbase: 16 swizzled key rows
template <int D, bool F16 = false>
LLM_DEVICE void qk_16keys(const uint32_t (&qa)[D / 16][4], uint32_t kbase, int lane, float (&s)[2][4]) {
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[nb][i] = 0.f;
    const int mat = lane >> 3, r = lane & 7;
    const int key = (mat >> 1) * 8 + r;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(tile_addr<D>(kbase, key, 2 * ks + (mat & 1)), b0, b1, b2, b3);
        mma_16<F16>(s[0], qa[ks], b0, b1);
        mma_16<F16>(s[1], qa[ks], b2, b3);
    }
}

// O(16 x D) += P(16 x 16 keys) V(16 keys x D)
template <int D, bool F16 = false>
LLM_DEVICE void pv_16keys(const uint32_t (&pa)[4], uint32_t vbase, int lane, float (&o)[D / 8][4]) {
    const int mat = lane >> 3, r = lane & 7;
    const int key = (mat & 1) * 8 + r;
#pragma unroll
    for (int c = 0; c < D / 16; ++c) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(tile_addr<D>(vbase, key, 2 * c + (mat >> 1)), b0, b1, b2, b3);
        mma_16<F16>(o[2 * c], pa, b0, b1);
        mma_16<F16>(o[2 * c + 1], pa, b2, b3);
    }
}

// ------------------------------------------------------------------------------------------------
// decode
// ------------------------------------------------------------------------------------------------
// Q8: the cache holds int8 rows + fp16 block scales (AttnDecodeParams).  The cp.async ring then carries the raw bytes (half
// the traffic) and the warp expands each 16-key sub-tile into one 16-bit work tile of the layout the MMAs read (fp16: see
// q8_unit_to_f16).
template <int D, bool Q8>
struct DecodeSmem {
    static constexpr int STAGES = Q8 ? 2 : 3;                // 8-bit: two raw stages keep the CTA small enough for three per SM
    static constexpr int SUB = 16 * D * 2;                   // bytes of a 16-key K (or V) sub-tile in 16-bit form
    static constexpr int RAW_SUB = 16 * D;                   // the same rows as int8
    static constexpr int RAW_SC = 16 * (D / 32) * 2;         // their block scales
    static constexpr int RAW_STAGE = 2 * (RAW_SUB + RAW_SC);
    static constexpr int PER_WARP = Q8 ? STAGES * RAW_STAGE + 2 * SUB : STAGES * 2 * SUB;
    static constexpr int MERGE = 4 * 16 * D * 4 + 4 * 16 * 2 * 4;
    static constexpr int BYTES = 4 * PER_WARP > MERGE ? 4 * PER_WARP : MERGE;
};

// 16 int8 values (four words) times one scale -> 16 fp16 (eight packed pairs), one PRMT and one HFMA2 per pair: a byte
// b ^ 0x80 under the high byte 0x64 is the fp16 number 1024 + 128 + x (fp16 carries 10 mantissa bits, so that is exact), and
// (1152 + x) * s - 1152 * s = x * s: the FMA is exact inside and 1152 * s is an fp16 number because the scales are stored
// with seven mantissa bits (rope_kv).  The 8-bit path therefore multiplies in fp16 (Q and the probabilities are converted
// to fp16 as well); sums stay in fp32.
LLM_DEVICE void q8_unit_to_f16(const uint4& w, __half2 sc2, __half2 off2, uint32_t (&o)[8]) {
    const uint32_t ws[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = __byte_perm(ws[k], 0x64646464u, 0x4140), hi = __byte_perm(ws[k], 0x64646464u, 0x4342);
        const __half2 r0 = __hfma2(*reinterpret_cast<const __half2*>(&lo), sc2, off2);
        const __half2 r1 = __hfma2(*reinterpret_cast<const __half2*>(&hi), sc2, off2);
        o[2 * k] = *reinterpret_cast<const uint32_t*>(&r0);
        o[2 * k + 1] = *reinterpret_cast<const uint32_t*>(&r1);
    }
}

template <int D, bool Q8>
__global__ void __launch_bounds__(128) paged_attn_decode_kernel(const AttnDecodeParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = blockIdx.x, split = blockIdx.y, seq = blockIdx.z;
    const int G = p.n_heads / p.n_kv_heads, R = p.rows_per_seq;
    const int seq_len = p.seq_lens[seq];
    const int n_pages = (seq_len + PAGE - 1) / PAGE;
    const int per = (n_pages + gridDim.y - 1) / gridDim.y;
    const int pg0 = split * per, pg1 = min(n_pages, pg0 + per);
    const int* btab = p.block_table + (size_t)seq * p.max_pages;
    using SM = DecodeSmem<D, Q8>;
    const uint32_t wbase = smem_u32(smem) + warp * SM::PER_WARP;
    const uint32_t work_k = wbase + SM::STAGES * SM::RAW_STAGE, work_v = work_k + SM::SUB;      // Q8 only: the expanded sub-tiles

    // Q fragments: MMA row i <-> (verify row r = i / G, q head g = i % G)
    uint32_t qa[D / 16][4];
    const int i0 = lane >> 2, i1 = i0 + 8;
    {
        const int cq = (lane & 3) * 2;
        auto qptr = [&](int i) -> const __nv_bfloat16* {
            if (i >= G * R) return nullptr;
            const int r = i / G, g = i % G;
            return p.q + ((size_t)(seq * R + r) * p.n_heads + kvh * G + g) * D;
        };
        const __nv_bfloat16 *q0 = qptr(i0), *q1 = qptr(i1);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int d0 = ks * 16 + cq;
            qa[ks][0] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + d0) : 0u;
            qa[ks][1] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + d0) : 0u;
            qa[ks][2] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + d0 + 8) : 0u;
            qa[ks][3] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + d0 + 8) : 0u;
            if (Q8) {
#pragma unroll
                for (int j = 0; j < 4; ++j) qa[ks][j] = pack_f16(bf16_lo(qa[ks][j]), bf16_hi(qa[ks][j]));
            }
        }
    }
    // causal limit per MMA row: verify row r sees keys < seq_len - (R - 1 - r)
    const int lim0 = (i0 < G * R) ? seq_len - (R - 1 - i0 / G) : 0;
    const int lim1 = (i1 < G * R) ? seq_len - (R - 1 - i1 / G) : 0;

    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const float sl2 = p.scale * 1.4426950408889634f;

    auto issue = [&](int pg, int stage) {
        if (Q8) {
            if (pg < pg1) {
                const size_t page = (size_t)LLM_CHECK_INDEX(btab[pg], p.n_pages);
                const uint8_t* pgp = reinterpret_cast<const uint8_t*>(p.kv) + page * p.page_bytes;
                const size_t rk = ((size_t)0 * p.n_kv_heads + kvh) * PAGE + (size_t)warp * 16, rv = ((size_t)1 * p.n_kv_heads + kvh) * PAGE + (size_t)warp * 16;
                const uint8_t *kp = pgp + rk * D, *vp = pgp + rv * D;
                const uint8_t *ks = pgp + p.scale_off + rk * (D / 32) * 2, *vs = pgp + p.scale_off + rv * (D / 32) * 2;
                const uint32_t rb = wbase + stage * SM::RAW_STAGE;        // [K rows][V rows][K scales][V scales]
#pragma unroll
                for (int t = 0; t < SM::RAW_SUB / 16 / 32; ++t) {
                    const int idx = t * 32 + lane;
                    cp_async16(rb + idx * 16, kp + idx * 16);
                    cp_async16(rb + SM::RAW_SUB + idx * 16, vp + idx * 16);
                }
                if (lane < SM::RAW_SC / 16) {
                    cp_async16(rb + 2 * SM::RAW_SUB + lane * 16, ks + lane * 16);
                    cp_async16(rb + 2 * SM::RAW_SUB + SM::RAW_SC + lane * 16, vs + lane * 16);
                }
            }
            cp_async_commit();
            return;
        }
        if (pg < pg1) {
            const size_t page = (size_t)LLM_CHECK_INDEX(btab[pg], p.n_pages);
            const __nv_bfloat16* kp = p.kv + ((page * 2 + 0) * p.n_kv_heads + kvh) * (size_t)(PAGE * D) + (size_t)warp * 16 * D;
            const __nv_bfloat16* vp = p.kv + ((page * 2 + 1) * p.n_kv_heads + kvh) * (size_t)(PAGE * D) + (size_t)warp * 16 * D;
            const uint32_t kb = wbase + stage * 2 * SM::SUB, vb = kb + SM::SUB;
            constexpr int UPR = D / 8;                    // 16-byte units per row
#pragma unroll
            for (int t = 0; t < 16 * UPR / 32; ++t) {
                const int idx = t * 32 + lane, row = idx / UPR, unit = idx % UPR;
                cp_async16(tile_addr<D>(kb, row, unit), kp + row * D + unit * 8);
                cp_async16(tile_addr<D>(vb, row, unit), vp + row * D + unit * 8);
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < SM::STAGES - 1; ++s) issue(pg0 + s, s);

    for (int pg = pg0; pg < pg1; ++pg) {
        const int stage = (pg - pg0) % SM::STAGES;
        issue(pg + SM::STAGES - 1, (pg - pg0 + SM::STAGES - 1) % SM::STAGES);
        cp_async_wait<SM::STAGES - 1>();
        __syncwarp();
        uint32_t kb = wbase + stage * 2 * SM::SUB, vb = kb + SM::SUB;
        if (Q8) {
            // expand this stage's raw rows into the work tiles: unit idx = 16 consecutive values of row idx / (D / 16)
            const uint32_t rb = wbase + stage * SM::RAW_STAGE;
            constexpr int UPR8 = D / 16, NU = 16 * UPR8 / 32;
            // all loads first (they pipeline in the shared-memory unit), then the arithmetic and the stores
            uint4 w[2][NU];
            uint16_t hs[2][NU];
#pragma unroll
            for (int t = 0; t < NU; ++t) {
                const int idx = t * 32 + lane, row = idx / UPR8, u = idx % UPR8;
#pragma unroll
                for (int kv = 0; kv < 2; ++kv) {
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[kv][t].x), "=r"(w[kv][t].y), "=r"(w[kv][t].z), "=r"(w[kv][t].w)
                                 : "r"(rb + kv * SM::RAW_SUB + idx * 16));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(hs[kv][t]) : "r"(rb + 2 * SM::RAW_SUB + kv * SM::RAW_SC + (row * (D / 32) + (u >> 1)) * 2));
                }
            }
#pragma unroll
            for (int t = 0; t < NU; ++t) {
                const int idx = t * 32 + lane, row = idx / UPR8, u = idx % UPR8;
#pragma unroll
                for (int kv = 0; kv < 2; ++kv) {
                    uint32_t o[8];
                    const __half hsc = __ushort_as_half(hs[kv][t]);
                    q8_unit_to_f16(w[kv][t], __half2half2(hsc), __half2half2(__hmul(hsc, __float2half_rn(-1152.0f))), o);
                    const uint32_t dst = kv ? work_v : work_k;
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(tile_addr<D>(dst, row, 2 * u)), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(tile_addr<D>(dst, row, 2 * u + 1)), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
                }
            }
            __syncwarp();
            kb = work_k; vb = work_v;
        }
        float s[2][4];
        qk_16keys<D, Q8>(qa, kb, lane, s);
        const int key0 = pg * PAGE + warp * 16 + (lane & 3) * 2;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + nb * 8 + e;
                s[nb][e] = key < lim0 ? s[nb][e] * sl2 : -INFINITY;
                s[nb][2 + e] = key < lim1 ? s[nb][2 + e] * sl2 : -INFINITY;
                mx0 = fmaxf(mx0, s[nb][e]);
                mx1 = fmaxf(mx1, s[nb][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
        const float base0 = nm0 == -INFINITY ? 0.f : nm0, base1 = nm1 == -INFINITY ? 0.f : nm1;
        const float c0 = exp2f(m0 - base0), c1 = exp2f(m1 - base1);
        m0 = nm0; m1 = nm1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[nb][e] = exp2f(s[nb][e] - base0); ps0 += s[nb][e];
                s[nb][2 + e] = exp2f(s[nb][2 + e] - base1); ps1 += s[nb][2 + e];
            }
        }
        l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
        uint32_t pa[4];
        if (Q8) {
            pa[0] = pack_f16(s[0][0], s[0][1]); pa[1] = pack_f16(s[0][2], s[0][3]);
            pa[2] = pack_f16(s[1][0], s[1][1]); pa[3] = pack_f16(s[1][2], s[1][3]);
        } else {
            pa[0] = pack_bf16(s[0][0], s[0][1]); pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[2] = pack_bf16(s[1][0], s[1][1]); pa[3] = pack_bf16(s[1][2], s[1][3]);
        }
        pv_16keys<D, Q8>(pa, vb, lane, o);
        __syncwarp();
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();

    // ---- merge the 4 warps (disjoint key subsets) through shared memory ----
    float* s_o = reinterpret_cast<float*>(smem);            // [4 warps][16 rows][D]
    float* s_ml = s_o + 4 * 16 * D;                          // [4][16][2]
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(&s_o[(warp * 16 + i0) * D + col]) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2*>(&s_o[(warp * 16 + i1) * D + col]) = make_float2(o[n][2], o[n][3]);
    }
    if ((lane & 3) == 0) {
        s_ml[(warp * 16 + i0) * 2] = m0; s_ml[(warp * 16 + i0) * 2 + 1] = l0;
        s_ml[(warp * 16 + i1) * 2] = m1; s_ml[(warp * 16 + i1) * 2 + 1] = l1;
    }
    __syncthreads();
    const int rows = G * R;
    // thread t handles column t % D of rows t / D, t / D + 128 / D, ...
    const int col = threadIdx.x % D;
    const size_t part_base = (((size_t)seq * p.n_kv_heads + kvh) * gridDim.y + split) * 16;
    for (int i = threadIdx.x / D; i < rows; i += 128 / D) {
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, s_ml[(w * 16 + i) * 2]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = s_ml[(w * 16 + i) * 2];
            const float c = mw == -INFINITY ? 0.f : exp2f(mw - m);
            l += c * s_ml[(w * 16 + i) * 2 + 1];
            acc += c * s_o[(w * 16 + i) * D + col];
        }
        if (gridDim.y == 1) {
            const int r = i / G, g = i % G;
            p.out[((size_t)(seq * R + r) * p.n_heads + kvh * G + g) * D + col] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
        } else {
            p.part_o[(part_base + i) * D + col] = acc;
            if (col == 0) { p.part_ml[(part_base + i) * 2] = m; p.part_ml[(part_base + i) * 2 + 1] = l; }
        }
    }
    if (gridDim.y == 1) return;

    // ---- last CTA of this (sequence, kv head) merges the splits ----
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(&p.tickets[seq * p.n_kv_heads + kvh], 1u);
        s_last = (t == gridDim.y - 1);
        if (s_last) p.tickets[seq * p.n_kv_heads + kvh] = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const size_t pb = (((size_t)seq * p.n_kv_heads + kvh) * gridDim.y) * 16;
    for (int i = threadIdx.x / D; i < rows; i += 128 / D) {
        float m = -INFINITY;
        for (int s = 0; s < (int)gridDim.y; ++s) m = fmaxf(m, __ldcg(&p.part_ml[(pb + s * 16 + i) * 2]));
        float l = 0.f, acc = 0.f;
        for (int s = 0; s < (int)gridDim.y; ++s) {
            const float ms = __ldcg(&p.part_ml[(pb + s * 16 + i) * 2]);
            const float c = ms == -INFINITY ? 0.f : exp2f(ms - m);
            l += c * __ldcg(&p.part_ml[(pb + s * 16 + i) * 2 + 1]);
            acc += c * __ldcg(&p.part_o[(pb + s * 16 + i) * D + col]);
        }
        const int r = i / G, g = i % G;
        p.out[((size_t)(seq * R + r) * p.n_heads + kvh * G + g) * D + col] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
    }
}

int attn_decode_pick_splits(int batch, int n_kv_heads, int max_pages_in_use) {
    int splits = (296 + batch * n_kv_heads - 1) / (batch * n_kv_heads);
    const int cap = (max_pages_in_use + 1) / 2;
    if (splits > cap) splits = cap;
    if (splits < 1) splits = 1;
    if (splits > 64) splits = 64;
    return splits;
}

cudaError_t launch_attn_decode(const AttnDecodeParams& p, int batch, int n_splits, cudaStream_t st) {
    const int G = p.n_heads / p.n_kv_heads;
    if (G * p.rows_per_seq > 16 || p.n_heads % p.n_kv_heads) return cudaErrorInvalidValue;
    dim3 grid(p.n_kv_heads, n_splits, batch);
    if (p.kv_q8 && (p.page_bytes % 16 || p.scale_off % 16)) return cudaErrorInvalidValue;     // 16-byte cp.async units
    auto go = [&](auto kernel, int smem) -> cudaError_t {
        static const void* done[8] = {};                     // kernels whose shared-memory limit has been raised
        const void* key = reinterpret_cast<const void*>(kernel);
        bool seen = false;
        for (const void* d : done) seen = seen || d == key;
        if (!seen) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return e;
            for (const void*& d : done) if (!d) { d = key; break; }
        }
        return launch_pdl(kernel, grid, dim3(128), smem, st, p);
    };
    constexpr int SLACK = 1024;
    if (p.head_dim == 128) {
        if (p.kv_q8) return go(paged_attn_decode_kernel<128, true>, DecodeSmem<128, true>::BYTES + SLACK);
        return go(paged_attn_decode_kernel<128, false>, DecodeSmem<128, false>::BYTES + SLACK);
    } else if (p.head_dim == 64) {
        if (p.kv_q8) return go(paged_attn_decode_kernel<64, true>, DecodeSmem<64, true>::BYTES + SLACK);
        return go(paged_attn_decode_kernel<64, false>, DecodeSmem<64, false>::BYTES + SLACK);
    }
    return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------------------------------
// prefill: 64 query rows per CTA, keys/values of one page per step
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) paged_attn_prefill_kernel(const AttnPrefillParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y, seq = blockIdx.z;
    const int G = p.n_heads / p.n_kv_heads, kvh = head / G;
    const int q_start = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_start;
    const int qt0 = blockIdx.x * 64;
    if (qt0 >= q_len) return;
    const int ctx = p.ctx_lens[seq];                 // tokens already in the cache before this chunk
    const int* btab = p.block_table + (size_t)seq * p.max_pages;
    constexpr int TILE = PAGE * D * 2;                // bytes of one K (or V) page tile
    const uint32_t sbase = smem_u32(smem);

    uint32_t qa[D / 16][4];
    const int r0 = qt0 + warp * 16 + (lane >> 2), r1 = r0 + 8;
    {
        const int cq = (lane & 3) * 2;
        const __nv_bfloat16* q0 = r0 < q_len ? p.q + ((size_t)(q_start + r0) * p.n_heads + head) * D : nullptr;
        const __nv_bfloat16* q1 = r1 < q_len ? p.q + ((size_t)(q_start + r1) * p.n_heads + head) * D : nullptr;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int d0 = ks * 16 + cq;
            qa[ks][0] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + d0) : 0u;
            qa[ks][1] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + d0) : 0u;
            qa[ks][2] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + d0 + 8) : 0u;
            qa[ks][3] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + d0 + 8) : 0u;
        }
    }
    const int lim0 = ctx + r0 + 1, lim1 = ctx + r1 + 1;           // row sees keys < lim
    const int kv_end = min(ctx + q_len, ctx + qt0 + 64);          // keys needed by this q tile
    const int n_pages = (kv_end + PAGE - 1) / PAGE;

    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const float sl2 = p.scale * 1.4426950408889634f;

    auto issue = [&](int pg, int stage) {
        if (pg < n_pages) {
            const size_t page = (size_t)LLM_CHECK_INDEX(btab[pg], p.n_pages);
            const __nv_bfloat16* kp = p.kv + ((page * 2 + 0) * p.n_kv_heads + kvh) * (size_t)(PAGE * D);
            const __nv_bfloat16* vp = p.kv + ((page * 2 + 1) * p.n_kv_heads + kvh) * (size_t)(PAGE * D);
            const uint32_t kb = sbase + stage * 2 * TILE, vb = kb + TILE;
            constexpr int UPR = D / 8;
#pragma unroll
            for (int t = 0; t < PAGE * UPR / 128; ++t) {
                const int idx = t * 128 + threadIdx.x, row = idx / UPR, unit = idx % UPR;
                cp_async16(tile_addr<D>(kb, row, unit), kp + row * D + unit * 8);
                cp_async16(tile_addr<D>(vb, row, unit), vp + row * D + unit * 8);
            }
        }
        cp_async_commit();
    };
    issue(0, 0);
    for (int pg = 0; pg < n_pages; ++pg) {
        const int stage = pg & 1;
        issue(pg + 1, stage ^ 1);
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t kb = sbase + stage * 2 * TILE, vb = kb + TILE;
        const bool need_mask = (pg + 1) * PAGE > ctx + qt0 + warp * 16 + 1;   // page reaches past this warp's first row
#pragma unroll
        for (int sub = 0; sub < PAGE / 16; ++sub) {
            const int key_base = pg * PAGE + sub * 16;
            if (key_base >= ctx + qt0 + warp * 16 + 16) break;                 // fully masked for every row of this warp
            float s[2][4];
            qk_16keys<D>(qa, kb + sub * 16 * D * 2, lane, s);
            const int key0 = key_base + (lane & 3) * 2;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key0 + nb * 8 + e;
                    s[nb][e] = (!need_mask || key < lim0) ? s[nb][e] * sl2 : -INFINITY;
                    s[nb][2 + e] = (!need_mask || key < lim1) ? s[nb][2 + e] * sl2 : -INFINITY;
                    mx0 = fmaxf(mx0, s[nb][e]);
                    mx1 = fmaxf(mx1, s[nb][2 + e]);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
            const float base0 = nm0 == -INFINITY ? 0.f : nm0, base1 = nm1 == -INFINITY ? 0.f : nm1;
            const float c0 = exp2f(m0 - base0), c1 = exp2f(m1 - base1);
            m0 = nm0; m1 = nm1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    s[nb][e] = exp2f(s[nb][e] - base0); ps0 += s[nb][e];
                    s[nb][2 + e] = exp2f(s[nb][2 + e] - base1); ps1 += s[nb][2 + e];
                }
            }
            l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;
#pragma unroll
            for (int n = 0; n < D / 8; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
            uint32_t pa[4];
            pa[0] = pack_bf16(s[0][0], s[0][1]); pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[2] = pack_bf16(s[1][0], s[1][1]); pa[3] = pack_bf16(s[1][2], s[1][3]);
            pv_16keys<D>(pa, vb + sub * 16 * D * 2, lane, o);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        if (r0 < q_len)
            *reinterpret_cast<uint32_t*>(p.out + ((size_t)(q_start + r0) * p.n_heads + head) * D + col) = pack_bf16(o[n][0] * inv0, o[n][1] * inv0);
        if (r1 < q_len)
            *reinterpret_cast<uint32_t*>(p.out + ((size_t)(q_start + r1) * p.n_heads + head) * D + col) = pack_bf16(o[n][2] * inv1, o[n][3] * inv1);
    }
}

cudaError_t launch_attn_prefill(const AttnPrefillParams& p, int n_seqs, int max_q_len, cudaStream_t st) {
    if (p.n_heads % p.n_kv_heads) return cudaErrorInvalidValue;
    dim3 grid((max_q_len + 63) / 64, p.n_heads, n_seqs);
    if (p.head_dim == 128) {
        constexpr int smem = 4 * PAGE * 128 * 2;
        static bool once = false;
        if (!once) { cudaFuncSetAttribute(paged_attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); once = true; }
        paged_attn_prefill_kernel<128><<<grid, 128, smem, st>>>(p);
    } else if (p.head_dim == 64) {
        constexpr int smem = 4 * PAGE * 64 * 2;
        paged_attn_prefill_kernel<64><<<grid, 128, smem, st>>>(p);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

LLM_DEFINE_BOUNDS_STATUS_READER(bounds_status_attention)

}  // namespace llm
