// Per-format access to weight chunks (128 rows x 256 columns, plane-separated; see ops/layout.py).
//
// Two families of device functions, both with lane == row inside a 32-row group:
//   dot_block<FMT, M>   integer dot product (dp4a) of one row's 256 weights with M int8-quantised
//                       activation rows; used by the small-batch GEMV.
//   dequant_block<FMT>  the row's 256 weights as bf16, emitted as 32 groups of 8 consecutive
//                       columns; used by the tensor-core GEMM's dequant warps, the embedding
//                       gather and the debug dequant kernel.
// The reference decodes the same formats into int8x4 groups for its dp4a / mma.sync kernels
// (reference: src/v2/kernels/cuda/gemm/CUDANativeVNNIDecodeCommon.cuh:265-452).
#pragma once
#include "common.cuh"

namespace llm {

enum Fmt : int { FMT_Q4_K = 0, FMT_Q5_K = 1, FMT_Q6_K = 2, FMT_Q8_0 = 3, FMT_Q4_0 = 4, FMT_IQ3_S = 5, FMT_COUNT = 6 };

template <int F> struct FmtTraits;
template <> struct FmtTraits<FMT_Q4_K>  { static constexpr int CHUNK = 128 * 144; static constexpr int P_QS = 0, P_META = 16384; };
template <> struct FmtTraits<FMT_Q5_K>  { static constexpr int CHUNK = 128 * 176; static constexpr int P_QS = 0, P_QH = 16384, P_META = 20480; };
template <> struct FmtTraits<FMT_Q6_K>  { static constexpr int CHUNK = 128 * 210; static constexpr int P_QL = 0, P_QH = 16384, P_SC = 24576, P_D = 26624; };
template <> struct FmtTraits<FMT_Q8_0>  { static constexpr int CHUNK = 128 * 272; static constexpr int P_QS = 0, P_D = 32768; };
template <> struct FmtTraits<FMT_Q4_0>  { static constexpr int CHUNK = 128 * 144; static constexpr int P_QS = 0, P_D = 16384; };
template <> struct FmtTraits<FMT_IQ3_S> { static constexpr int CHUNK = 128 * 110; static constexpr int P_QS = 0, P_SIGNS = 8192, P_QH = 12288, P_SC = 13312, P_D = 13824; };

__host__ __device__ inline int fmt_chunk_bytes(int fmt) {
    switch (fmt) {
        case FMT_Q4_K: return FmtTraits<FMT_Q4_K>::CHUNK;
        case FMT_Q5_K: return FmtTraits<FMT_Q5_K>::CHUNK;
        case FMT_Q6_K: return FmtTraits<FMT_Q6_K>::CHUNK;
        case FMT_Q8_0: return FmtTraits<FMT_Q8_0>::CHUNK;
        case FMT_Q4_0: return FmtTraits<FMT_Q4_0>::CHUNK;
        case FMT_IQ3_S: return FmtTraits<FMT_IQ3_S>::CHUNK;
    }
    return 0;
}

// IQ3_S codebook: 512 entries, four unsigned magnitudes per entry (one copy per translation unit).
static __device__ const uint32_t g_iq3s_grid[512] = {
#include "iq3s_grid.inc"
};

// 16-byte unit `u` of a plane with U units per row, row group g, lane = row in group.
LLM_DEVICE const uint8_t* unit_ptr(const uint8_t* plane, int U, int g, int u, int lane) {
    return plane + (((g * U + u) * 32 + lane) << 4);
}

// ---- K-quant 6-bit scale/min unpack (12 packed bytes in words s0,s1,s2) -------------------------
LLM_DEVICE void unpack_k4_scales(uint32_t s0, uint32_t s1, uint32_t s2, int (&sc)[8], int (&mn)[8]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t a = (s0 >> (8 * j)) & 0xff, b = (s1 >> (8 * j)) & 0xff, c = (s2 >> (8 * j)) & 0xff;
        sc[j] = a & 63;
        mn[j] = b & 63;
        sc[j + 4] = (c & 0xf) | ((a >> 6) << 4);
        mn[j + 4] = (c >> 4) | ((b >> 6) << 4);
    }
}

// Expand the low 4 bits of x into a byte mask (0xff where the bit is set).
LLM_DEVICE uint32_t expand4(uint32_t x) { return (((x & 0xf) * 0x00204081u) & 0x01010101u) * 0xffu; }

// =================================================================================================
// GEMV side: int8 activations.  One ActBlk per (activation row, 256-column block).
// =================================================================================================
struct __align__(16) ActBlk {
    int a[64];        // 256 int8 values
    float d[8];       // scale of each 32-element block
    float ds16[16];   // d * (sum of the int8 values) per 16 elements
};

LLM_DEVICE int dp4a_u(uint32_t a, int b, int c) {   // a: four unsigned bytes, b: four signed bytes
    int r;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
LLM_DEVICE int dp4a_s(uint32_t a, int b, int c) {   // both signed
    int r;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// Where a chunk is read from: global memory (read-only path, no L1 allocation) or a copy in shared memory (a generic
// pointer into the CTA's shared window).  The dot products below are written once against this policy.
struct LdGlobalNc {
    LLM_DEVICE static uint4 v4(const void* p) { return ldg_nc_v4(p); }
    LLM_DEVICE static uint2 v2(const void* p) { return ldg_nc_v2(p); }
    LLM_DEVICE static uint32_t u32(const void* p) { return ldg_nc_u32(p); }
    LLM_DEVICE static uint16_t u16(const void* p) { return ldg_nc_u16(p); }
};
struct LdShared {
    LLM_DEVICE static uint32_t a(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
    LLM_DEVICE static uint4 v4(const void* p) {
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a(p)));
        return v;
    }
    LLM_DEVICE static uint2 v2(const void* p) {
        uint2 v;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a(p)));
        return v;
    }
    LLM_DEVICE static uint32_t u32(const void* p) {
        uint32_t v;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a(p)));
        return v;
    }
    LLM_DEVICE static uint16_t u16(const void* p) {
        uint16_t v;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a(p)));
        return v;
    }
};
template <int F, int M, class L = LdGlobalNc> struct DotBlock;

template <int M, class L> struct DotBlock<FMT_Q4_K, M, L> {
    LLM_DEVICE static void run(const uint8_t* chunk, int g, int lane, const ActBlk* act, int act_stride, float (&acc)[M]) {
        using T = FmtTraits<FMT_Q4_K>;
        const uint4 meta = L::v4(chunk + T::P_META + ((g * 32 + lane) << 4));
        uint4 w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = L::v4(unit_ptr(chunk + T::P_QS, 8, g, u, lane));
        const float d = half_bits_to_float(meta.x & 0xffff), dmin = half_bits_to_float(meta.x >> 16);
        int sc[8], mn[8];
        unpack_k4_scales(meta.y, meta.z, meta.w, sc, mn);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int lo[M], hi[M];
#pragma unroll
            for (int m = 0; m < M; ++m) lo[m] = hi[m] = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 q = w[2 * j + h];
                const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const ActBlk& ab = *reinterpret_cast<const ActBlk*>(reinterpret_cast<const uint8_t*>(act) + m * act_stride);
                    const int4 al = *reinterpret_cast<const int4*>(&ab.a[16 * j + 4 * h]);
                    const int4 ah = *reinterpret_cast<const int4*>(&ab.a[16 * j + 8 + 4 * h]);
                    const int as_l[4] = {al.x, al.y, al.z, al.w}, as_h[4] = {ah.x, ah.y, ah.z, ah.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        lo[m] = dp4a_u(ws[i] & 0x0f0f0f0fu, as_l[i], lo[m]);
                        hi[m] = dp4a_u((ws[i] >> 4) & 0x0f0f0f0fu, as_h[i], hi[m]);
                    }
                }
            }
            const float s_lo = d * sc[2 * j], s_hi = d * sc[2 * j + 1];
            const float m_lo = dmin * mn[2 * j], m_hi = dmin * mn[2 * j + 1];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const ActBlk& ab = *reinterpret_cast<const ActBlk*>(reinterpret_cast<const uint8_t*>(act) + m * act_stride);
                acc[m] += s_lo * (ab.d[2 * j] * lo[m]) - m_lo * (ab.ds16[4 * j] + ab.ds16[4 * j + 1]);
                acc[m] += s_hi * (ab.d[2 * j + 1] * hi[m]) - m_hi * (ab.ds16[4 * j + 2] + ab.ds16[4 * j + 3]);
            }
        }
    }
};

template <int M, class L> struct DotBlock<FMT_Q5_K, M, L> {
    LLM_DEVICE static void run(const uint8_t* chunk, int g, int lane, const ActBlk* act, int act_stride, float (&acc)[M]) {
        using T = FmtTraits<FMT_Q5_K>;
        const uint4 meta = L::v4(chunk + T::P_META + ((g * 32 + lane) << 4));
        uint4 w[8], qh[2];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = L::v4(unit_ptr(chunk + T::P_QS, 8, g, u, lane));
#pragma unroll
        for (int u = 0; u < 2; ++u) qh[u] = L::v4(unit_ptr(chunk + T::P_QH, 2, g, u, lane));
        const float d = half_bits_to_float(meta.x & 0xffff), dmin = half_bits_to_float(meta.x >> 16);
        int sc[8], mn[8];
        unpack_k4_scales(meta.y, meta.z, meta.w, sc, mn);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int lo[M], hi[M];
#pragma unroll
            for (int m = 0; m < M; ++m) lo[m] = hi[m] = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 q = w[2 * j + h];
                const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
                const uint32_t hs[4] = {qh[h].x, qh[h].y, qh[h].z, qh[h].w};
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const ActBlk& ab = *reinterpret_cast<const ActBlk*>(reinterpret_cast<const uint8_t*>(act) + m * act_stride);
                    const int4 al = *reinterpret_cast<const int4*>(&ab.a[16 * j + 4 * h]);
                    const int4 ah = *reinterpret_cast<const int4*>(&ab.a[16 * j + 8 + 4 * h]);
                    const int as_l[4] = {al.x, al.y, al.z, al.w}, as_h[4] = {ah.x, ah.y, ah.z, ah.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t ql = (ws[i] & 0x0f0f0f0fu) | (((hs[i] >> (2 * j)) & 0x01010101u) << 4);
                        const uint32_t qu = ((ws[i] >> 4) & 0x0f0f0f0fu) | (((hs[i] >> (2 * j + 1)) & 0x01010101u) << 4);
                        lo[m] = dp4a_u(ql, as_l[i], lo[m]);
                        hi[m] = dp4a_u(qu, as_h[i], hi[m]);
                    }
                }
            }
            const float s_lo = d * sc[2 * j], s_hi = d * sc[2 * j + 1];
            const float m_lo = dmin * mn[2 * j], m_hi = dmin * mn[2 * j + 1];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const ActBlk& ab = *reinterpret_cast<const ActBlk*>(reinterpret_cast<const uint8_t*>(act) + m * act_stride);
                acc[m] += s_lo * (ab.d[2 * j] * lo[m]) - m_lo * (ab.ds16[4 * j] + ab.ds16[4 * j + 1]);
                acc[m] += s_hi * (ab.d[2 * j + 1] * hi[m]) - m_hi * (ab.ds16[4 * j + 2] + ab.ds16[4 * j + 3]);
            }
        }
    }
};

template <int M, class L> struct DotBlock<FMT_Q6_K, M, L> {
    LLM_DEVICE static void run(const uint8_t* chunk, int g, int lane, const ActBlk* act, int act_stride, float (&acc)[M]) {
        using T = FmtTraits<FMT_Q6_K>;
        const int row = g * 32 + lane;
        const uint4 scw = L::v4(chunk + T::P_SC + (row << 4));
        const float d = half_bits_to_float(L::u16(chunk + T::P_D + (row << 1)));
        uint4 ql[8], qh[4];
#pragma unroll
        for (int u = 0; u < 8; ++u) ql[u] = L::v4(unit_ptr(chunk + T::P_QL, 8, g, u, lane));
#pragma unroll
        for (int u = 0; u < 4; ++u) qh[u] = L::v4(unit_ptr(chunk + T::P_QH, 4, g, u, lane));
        const uint32_t scs[4] = {scw.x, scw.y, scw.z, scw.w};
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int lh = 0; lh < 2; ++lh) {
                const uint4 A = ql[4 * n + lh], B = ql[4 * n + 2 + lh], H = qh[2 * n + lh];
                const uint32_t as_[4] = {A.x, A.y, A.z, A.w}, bs_[4] = {B.x, B.y, B.z, B.w}, hs_[4] = {H.x, H.y, H.z, H.w};
                uint32_t q1[4], q2[4], q3[4], q4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    q1[i] = (as_[i] & 0x0f0f0f0fu) | ((hs_[i] << 4) & 0x30303030u);
                    q2[i] = (bs_[i] & 0x0f0f0f0fu) | ((hs_[i] << 2) & 0x30303030u);
                    q3[i] = ((as_[i] >> 4) & 0x0f0f0f0fu) | (hs_[i] & 0x30303030u);
                    q4[i] = ((bs_[i] >> 4) & 0x0f0f0f0fu) | ((hs_[i] >> 2) & 0x30303030u);
                }
                // sub-block (16 columns) indices of q1..q4 and their int8 scales
                const int s1 = 8 * n + lh, s2 = s1 + 2, s3 = s1 + 4, s4 = s1 + 6;
                const float f1 = d * static_cast<int8_t>((scs[s1 >> 2] >> (8 * (s1 & 3))) & 0xff);
                const float f2 = d * static_cast<int8_t>((scs[s2 >> 2] >> (8 * (s2 & 3))) & 0xff);
                const float f3 = d * static_cast<int8_t>((scs[s3 >> 2] >> (8 * (s3 & 3))) & 0xff);
                const float f4 = d * static_cast<int8_t>((scs[s4 >> 2] >> (8 * (s4 & 3))) & 0xff);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const ActBlk& ab = *reinterpret_cast<const ActBlk*>(reinterpret_cast<const uint8_t*>(act) + m * act_stride);
                    const int base = 32 * n + 4 * lh;   // int index of column 128n + 16lh
                    const int4 a1 = *reinterpret_cast<const int4*>(&ab.a[base]);
                    const int4 a2 = *reinterpret_cast<const int4*>(&ab.a[base + 8]);
                    const int4 a3 = *reinterpret_cast<const int4*>(&ab.a[base + 16]);
                    const int4 a4 = *reinterpret_cast<const int4*>(&ab.a[base + 24]);
                    int i1 = 0, i2 = 0, i3 = 0, i4 = 0;
                    i1 = dp4a_u(q1[0], a1.x, i1); i1 = dp4a_u(q1[1], a1.y, i1); i1 = dp4a_u(q1[2], a1.z, i1); i1 = dp4a_u(q1[3], a1.w, i1);
                    i2 = dp4a_u(q2[0], a2.x, i2); i2 = dp4a_u(q2[1], a2.y, i2); i2 = dp4a_u(q2[2], a2.z, i2); i2 = dp4a_u(q2[3], a2.w, i2);
                    i3 = dp4a_u(q3[0], a3.x, i3); i3 = dp4a_u(q3[1], a3.y, i3); i3 = dp4a_u(q3[2], a3.z, i3); i3 = dp4a_u(q3[3], a3.w, i3);
                    i4 = dp4a_u(q4[0], a4.x, i4); i4 = dp4a_u(q4[1], a4.y, i4); i4 = dp4a_u(q4[2], a4.z, i4); i4 = dp4a_u(q4[3], a4.w, i4);
                    acc[m] += f1 * (ab.d[s1 >> 1] * i1 - 32.0f * ab.ds16[s1]);
                    acc[m] += f2 * (ab.d[s2 >> 1] * i2 - 32.0f * ab.ds16[s2]);
                    acc[m] += f3 * (ab.d[s3 >> 1] * i3 - 32.0f * ab.ds16[s3]);
                    acc[m] += f4 * (ab.d[s4 >> 1] * i4 - 32.0f * ab.ds16[s4]);
                }
            }
        }
    }
};

template <int M, class L> struct DotBlock<FMT_Q8_0, M, L> {
    LLM_DEVICE static void run(const uint8_t* chunk, int g, int lane, const ActBlk* act, int act_stride, float (&acc)[M]) {
        using T = FmtTraits<FMT_Q8_0>;
        const uint4 dw = L::v4(chunk + T::P_D + ((g * 32 + lane) << 4));
        const uint32_t ds[4] = {dw.x, dw.y, dw.z, dw.w};
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const uint4 q0 = L::v4(unit_ptr(chunk + T::P_QS, 16, g, 2 * b, lane));
            const uint4 q1 = L::v4(unit_ptr(chunk + T::P_QS, 16, g, 2 * b + 1, lane));
            const float d = half_bits_to_float((ds[b >> 1] >> (16 * (b & 1))) & 0xffff);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const ActBlk& ab = *reinterpret_cast<const ActBlk*>(reinterpret_cast<const uint8_t*>(act) + m * act_stride);
                const int4 a0 = *reinterpret_cast<const int4*>(&ab.a[8 * b]);
                const int4 a1 = *reinterpret_cast<const int4*>(&ab.a[8 * b + 4]);
                int s = 0;
                s = dp4a_s(q0.x, a0.x, s); s = dp4a_s(q0.y, a0.y, s); s = dp4a_s(q0.z, a0.z, s); s = dp4a_s(q0.w, a0.w, s);
                s = dp4a_s(q1.x, a1.x, s); s = dp4a_s(q1.y, a1.y, s); s = dp4a_s(q1.z, a1.z, s); s = dp4a_s(q1.w, a1.w, s);
                acc[m] += d * (ab.d[b] * s);
            }
        }
    }
};

template <int M, class L> struct DotBlock<FMT_Q4_0, M, L> {
    LLM_DEVICE static void run(const uint8_t* chunk, int g, int lane, const ActBlk* act, int act_stride, float (&acc)[M]) {
        using T = FmtTraits<FMT_Q4_0>;
        const uint4 dw = L::v4(chunk + T::P_D + ((g * 32 + lane) << 4));
        const uint32_t ds[4] = {dw.x, dw.y, dw.z, dw.w};
        uint4 w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = L::v4(unit_ptr(chunk + T::P_QS, 8, g, u, lane));
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const uint32_t ws[4] = {w[b].x, w[b].y, w[b].z, w[b].w};
            const float d = half_bits_to_float((ds[b >> 1] >> (16 * (b & 1))) & 0xffff);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const ActBlk& ab = *reinterpret_cast<const ActBlk*>(reinterpret_cast<const uint8_t*>(act) + m * act_stride);
                const int4 al = *reinterpret_cast<const int4*>(&ab.a[8 * b]);
                const int4 ah = *reinterpret_cast<const int4*>(&ab.a[8 * b + 4]);
                const int as_l[4] = {al.x, al.y, al.z, al.w}, as_h[4] = {ah.x, ah.y, ah.z, ah.w};
                int s = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s = dp4a_u(ws[i] & 0x0f0f0f0fu, as_l[i], s);
                    s = dp4a_u((ws[i] >> 4) & 0x0f0f0f0fu, as_h[i], s);
                }
                acc[m] += d * (ab.d[b] * s - 8.0f * (ab.ds16[2 * b] + ab.ds16[2 * b + 1]));
            }
        }
    }
};

template <int M, class L> struct DotBlock<FMT_IQ3_S, M, L> {
    // `grid` must point at a shared-memory copy of g_iq3s_grid.
    LLM_DEVICE static void run(const uint8_t* chunk, int g, int lane, const ActBlk* act, int act_stride, float (&acc)[M],
                               const uint32_t* grid) {
        using T = FmtTraits<FMT_IQ3_S>;
        const int row = g * 32 + lane;
        uint4 qs[4], sg[2];
#pragma unroll
        for (int u = 0; u < 4; ++u) qs[u] = L::v4(unit_ptr(chunk + T::P_QS, 4, g, u, lane));
#pragma unroll
        for (int u = 0; u < 2; ++u) sg[u] = L::v4(unit_ptr(chunk + T::P_SIGNS, 2, g, u, lane));
        const uint2 qh = L::v2(chunk + T::P_QH + (row << 3));
        const uint32_t scw = L::u32(chunk + T::P_SC + (row << 2));
        const float d = half_bits_to_float(L::u16(chunk + T::P_D + (row << 1)));
#pragma unroll
        for (int ib = 0; ib < 8; ++ib) {
            const uint4 q4 = qs[ib >> 1];
            const uint32_t qa = (ib & 1) ? q4.z : q4.x, qb = (ib & 1) ? q4.w : q4.y;   // 8 index bytes
            const uint32_t hb = ((ib < 4 ? qh.x : qh.y) >> (8 * (ib & 3))) & 0xff;
            const uint4 s4 = sg[ib >> 2];
            const uint32_t sw = (ib & 3) == 0 ? s4.x : (ib & 3) == 1 ? s4.y : (ib & 3) == 2 ? s4.z : s4.w;
            uint32_t v[8];
#pragma unroll
            for (int l = 0; l < 4; ++l) {
                const uint32_t pair = (l < 2 ? qa : qb) >> (16 * (l & 1));
                const uint32_t i1 = (pair & 0xff) | ((hb << (8 - 2 * l)) & 256);
                const uint32_t i2 = ((pair >> 8) & 0xff) | ((hb << (7 - 2 * l)) & 256);
                const uint32_t sbyte = (sw >> (8 * l)) & 0xff;
                const uint32_t m1 = expand4(sbyte), m2 = expand4(sbyte >> 4);
                v[2 * l] = __vsub4(grid[i1] ^ m1, m1);
                v[2 * l + 1] = __vsub4(grid[i2] ^ m2, m2);
            }
            const float db = d * (1 + 2 * ((scw >> (4 * ib)) & 0xf));
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const ActBlk& ab = *reinterpret_cast<const ActBlk*>(reinterpret_cast<const uint8_t*>(act) + m * act_stride);
                const int4 a0 = *reinterpret_cast<const int4*>(&ab.a[8 * ib]);
                const int4 a1 = *reinterpret_cast<const int4*>(&ab.a[8 * ib + 4]);
                int s = 0;
                s = dp4a_s(v[0], a0.x, s); s = dp4a_s(v[1], a0.y, s); s = dp4a_s(v[2], a0.z, s); s = dp4a_s(v[3], a0.w, s);
                s = dp4a_s(v[4], a1.x, s); s = dp4a_s(v[5], a1.y, s); s = dp4a_s(v[6], a1.z, s); s = dp4a_s(v[7], a1.w, s);
                acc[m] += db * (ab.d[ib] * s);
            }
        }
    }
};

// =================================================================================================
// Dequant side: bf16 output, 8 consecutive columns per emit.
// =================================================================================================
// bytes (b0,b1) of `w`, each < 128, -> bf16x2 {128 + b0, 128 + b1} (exact: bf16 has 8 significant bits)
LLM_DEVICE uint32_t magic_pair01(uint32_t w) { return __byte_perm(w, 0x43434343u, 0x4140); }
LLM_DEVICE uint32_t magic_pair23(uint32_t w) { return __byte_perm(w, 0x43434343u, 0x4342); }

LLM_DEVICE __nv_bfloat162 as_bf162(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }
LLM_DEVICE uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// (bytes - offset) * scale + bias for 4 bytes of w (each < 128) -> two bf16x2 words
LLM_DEVICE void affine4(uint32_t w, __nv_bfloat162 offset, __nv_bfloat162 scale, __nv_bfloat162 bias, uint32_t& o0, uint32_t& o1) {
    o0 = as_u32(__hfma2(__hsub2(as_bf162(magic_pair01(w)), offset), scale, bias));
    o1 = as_u32(__hfma2(__hsub2(as_bf162(magic_pair23(w)), offset), scale, bias));
}

template <int F> struct DequantBlock;
// Each format offers
//   Regs  load(chunk, g, lane)            the row's packed bytes, fetched into registers
//   void  process(regs, sink[, grid])     bf16 conversion; the sink receives
//           sink.begin(atom, n)           before the first group of 64-column atoms [atom, atom+n)
//           sink.emit(kgroup, uint4)      8 consecutive columns 8*kgroup .. 8*kgroup+7
//           sink.end(atom, n)             after the last group of those atoms
// Atoms are produced in ascending order, which lets a GEMM release them to the MMA one by one.

template <> struct DequantBlock<FMT_Q4_K> {
    struct Regs { uint4 meta; uint4 q[8]; };
    LLM_DEVICE static Regs load(const uint8_t* chunk, int g, int lane) {
        using T = FmtTraits<FMT_Q4_K>;
        Regs r;
        r.meta = ldg_nc_v4(chunk + T::P_META + ((g * 32 + lane) << 4));
#pragma unroll
        for (int u = 0; u < 8; ++u) r.q[u] = ldg_nc_v4(unit_ptr(chunk + T::P_QS, 8, g, u, lane));
        return r;
    }
    template <class S> LLM_DEVICE static void process(const Regs& r, S& sink) {
        const float d = half_bits_to_float(r.meta.x & 0xffff), dmin = half_bits_to_float(r.meta.x >> 16);
        int sc[8], mn[8];
        unpack_k4_scales(r.meta.y, r.meta.z, r.meta.w, sc, mn);
        const __nv_bfloat162 off = __float2bfloat162_rn(128.0f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sink.begin(j, 1);
            const __nv_bfloat162 s_lo = __float2bfloat162_rn(d * sc[2 * j]), b_lo = __float2bfloat162_rn(-dmin * mn[2 * j]);
            const __nv_bfloat162 s_hi = __float2bfloat162_rn(d * sc[2 * j + 1]), b_hi = __float2bfloat162_rn(-dmin * mn[2 * j + 1]);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 q = r.q[2 * j + h];
                uint4 o;
                affine4(q.x & 0x0f0f0f0fu, off, s_lo, b_lo, o.x, o.y);
                affine4(q.y & 0x0f0f0f0fu, off, s_lo, b_lo, o.z, o.w);
                sink.emit(8 * j + 2 * h, o);
                affine4(q.z & 0x0f0f0f0fu, off, s_lo, b_lo, o.x, o.y);
                affine4(q.w & 0x0f0f0f0fu, off, s_lo, b_lo, o.z, o.w);
                sink.emit(8 * j + 2 * h + 1, o);
                affine4((q.x >> 4) & 0x0f0f0f0fu, off, s_hi, b_hi, o.x, o.y);
                affine4((q.y >> 4) & 0x0f0f0f0fu, off, s_hi, b_hi, o.z, o.w);
                sink.emit(8 * j + 4 + 2 * h, o);
                affine4((q.z >> 4) & 0x0f0f0f0fu, off, s_hi, b_hi, o.x, o.y);
                affine4((q.w >> 4) & 0x0f0f0f0fu, off, s_hi, b_hi, o.z, o.w);
                sink.emit(8 * j + 4 + 2 * h + 1, o);
            }
            sink.end(j, 1);
        }
    }
};

template <> struct DequantBlock<FMT_Q5_K> {
    struct Regs { uint4 meta; uint4 q[8]; uint4 qh[2]; };
    LLM_DEVICE static Regs load(const uint8_t* chunk, int g, int lane) {
        using T = FmtTraits<FMT_Q5_K>;
        Regs r;
        r.meta = ldg_nc_v4(chunk + T::P_META + ((g * 32 + lane) << 4));
#pragma unroll
        for (int u = 0; u < 8; ++u) r.q[u] = ldg_nc_v4(unit_ptr(chunk + T::P_QS, 8, g, u, lane));
        r.qh[0] = ldg_nc_v4(unit_ptr(chunk + T::P_QH, 2, g, 0, lane));
        r.qh[1] = ldg_nc_v4(unit_ptr(chunk + T::P_QH, 2, g, 1, lane));
        return r;
    }
    template <class S> LLM_DEVICE static void process(const Regs& r, S& sink) {
        const float d = half_bits_to_float(r.meta.x & 0xffff), dmin = half_bits_to_float(r.meta.x >> 16);
        int sc[8], mn[8];
        unpack_k4_scales(r.meta.y, r.meta.z, r.meta.w, sc, mn);
        const __nv_bfloat162 off = __float2bfloat162_rn(128.0f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sink.begin(j, 1);
            const __nv_bfloat162 s_lo = __float2bfloat162_rn(d * sc[2 * j]), b_lo = __float2bfloat162_rn(-dmin * mn[2 * j]);
            const __nv_bfloat162 s_hi = __float2bfloat162_rn(d * sc[2 * j + 1]), b_hi = __float2bfloat162_rn(-dmin * mn[2 * j + 1]);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 q = r.q[2 * j + h];
                const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
                const uint32_t hs[4] = {r.qh[h].x, r.qh[h].y, r.qh[h].z, r.qh[h].w};
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    lo[i] = (ws[i] & 0x0f0f0f0fu) | (((hs[i] >> (2 * j)) & 0x01010101u) << 4);
                    hi[i] = ((ws[i] >> 4) & 0x0f0f0f0fu) | (((hs[i] >> (2 * j + 1)) & 0x01010101u) << 4);
                }
                uint4 o;
                affine4(lo[0], off, s_lo, b_lo, o.x, o.y); affine4(lo[1], off, s_lo, b_lo, o.z, o.w);
                sink.emit(8 * j + 2 * h, o);
                affine4(lo[2], off, s_lo, b_lo, o.x, o.y); affine4(lo[3], off, s_lo, b_lo, o.z, o.w);
                sink.emit(8 * j + 2 * h + 1, o);
                affine4(hi[0], off, s_hi, b_hi, o.x, o.y); affine4(hi[1], off, s_hi, b_hi, o.z, o.w);
                sink.emit(8 * j + 4 + 2 * h, o);
                affine4(hi[2], off, s_hi, b_hi, o.x, o.y); affine4(hi[3], off, s_hi, b_hi, o.z, o.w);
                sink.emit(8 * j + 4 + 2 * h + 1, o);
            }
            sink.end(j, 1);
        }
    }
};

template <> struct DequantBlock<FMT_Q6_K> {
    struct Regs { uint4 sc; uint32_t d; uint4 ql[8]; uint4 qh[4]; };
    LLM_DEVICE static Regs load(const uint8_t* chunk, int g, int lane) {
        using T = FmtTraits<FMT_Q6_K>;
        const int row = g * 32 + lane;
        Regs r;
        r.sc = ldg_nc_v4(chunk + T::P_SC + (row << 4));
        r.d = ldg_nc_u16(chunk + T::P_D + (row << 1));
#pragma unroll
        for (int u = 0; u < 8; ++u) r.ql[u] = ldg_nc_v4(unit_ptr(chunk + T::P_QL, 8, g, u, lane));
#pragma unroll
        for (int u = 0; u < 4; ++u) r.qh[u] = ldg_nc_v4(unit_ptr(chunk + T::P_QH, 4, g, u, lane));
        return r;
    }
    template <class S> LLM_DEVICE static void process(const Regs& r, S& sink) {
        const uint32_t scs[4] = {r.sc.x, r.sc.y, r.sc.z, r.sc.w};
        const float d = half_bits_to_float((uint16_t)r.d);
        const __nv_bfloat162 off = __float2bfloat162_rn(160.0f), zero = __float2bfloat162_rn(0.0f);
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            sink.begin(2 * n, 2);
#pragma unroll
            for (int lh = 0; lh < 2; ++lh) {
                const uint4 A = r.ql[4 * n + lh], B = r.ql[4 * n + 2 + lh], H = r.qh[2 * n + lh];
                const uint32_t as_[4] = {A.x, A.y, A.z, A.w}, bs_[4] = {B.x, B.y, B.z, B.w}, hs_[4] = {H.x, H.y, H.z, H.w};
                const int s1 = 8 * n + lh;
                __nv_bfloat162 f[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int s = s1 + 2 * t;
                    f[t] = __float2bfloat162_rn(d * static_cast<int8_t>((scs[s >> 2] >> (8 * (s & 3))) & 0xff));
                }
                uint32_t q[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    q[0][i] = (as_[i] & 0x0f0f0f0fu) | ((hs_[i] << 4) & 0x30303030u);
                    q[1][i] = (bs_[i] & 0x0f0f0f0fu) | ((hs_[i] << 2) & 0x30303030u);
                    q[2][i] = ((as_[i] >> 4) & 0x0f0f0f0fu) | (hs_[i] & 0x30303030u);
                    q[3][i] = ((bs_[i] >> 4) & 0x0f0f0f0fu) | ((hs_[i] >> 2) & 0x30303030u);
                }
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int kg = 16 * n + 4 * t + 2 * lh;      // columns 128n + 32t + 16lh + [0,16)
                    uint4 o;
                    affine4(q[t][0], off, f[t], zero, o.x, o.y); affine4(q[t][1], off, f[t], zero, o.z, o.w);
                    sink.emit(kg, o);
                    affine4(q[t][2], off, f[t], zero, o.x, o.y); affine4(q[t][3], off, f[t], zero, o.z, o.w);
                    sink.emit(kg + 1, o);
                }
            }
            sink.end(2 * n, 2);
        }
    }
};

template <> struct DequantBlock<FMT_Q8_0> {
    struct Regs { uint4 d; uint4 q[16]; };
    LLM_DEVICE static Regs load(const uint8_t* chunk, int g, int lane) {
        using T = FmtTraits<FMT_Q8_0>;
        Regs r;
        r.d = ldg_nc_v4(chunk + T::P_D + ((g * 32 + lane) << 4));
#pragma unroll
        for (int u = 0; u < 16; ++u) r.q[u] = ldg_nc_v4(unit_ptr(chunk + T::P_QS, 16, g, u, lane));
        return r;
    }
    template <class S> LLM_DEVICE static void process(const Regs& r, S& sink) {
        const uint32_t ds[4] = {r.d.x, r.d.y, r.d.z, r.d.w};
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            sink.begin(a, 1);
#pragma unroll
            for (int uu = 0; uu < 4; ++uu) {
                const int u = 4 * a + uu, b = u >> 1;
                const float d = half_bits_to_float((ds[b >> 1] >> (16 * (b & 1))) & 0xffff);
                const uint32_t ws[4] = {r.q[u].x, r.q[u].y, r.q[u].z, r.q[u].w};
                uint32_t o[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float v0 = d * static_cast<int8_t>(ws[i] & 0xff), v1 = d * static_cast<int8_t>((ws[i] >> 8) & 0xff);
                    const float v2 = d * static_cast<int8_t>((ws[i] >> 16) & 0xff), v3 = d * static_cast<int8_t>(ws[i] >> 24);
                    o[2 * i] = pack_bf16(v0, v1);
                    o[2 * i + 1] = pack_bf16(v2, v3);
                }
                sink.emit(2 * u, make_uint4(o[0], o[1], o[2], o[3]));
                sink.emit(2 * u + 1, make_uint4(o[4], o[5], o[6], o[7]));
            }
            sink.end(a, 1);
        }
    }
};

template <> struct DequantBlock<FMT_Q4_0> {
    struct Regs { uint4 d; uint4 q[8]; };
    LLM_DEVICE static Regs load(const uint8_t* chunk, int g, int lane) {
        using T = FmtTraits<FMT_Q4_0>;
        Regs r;
        r.d = ldg_nc_v4(chunk + T::P_D + ((g * 32 + lane) << 4));
#pragma unroll
        for (int u = 0; u < 8; ++u) r.q[u] = ldg_nc_v4(unit_ptr(chunk + T::P_QS, 8, g, u, lane));
        return r;
    }
    template <class S> LLM_DEVICE static void process(const Regs& r, S& sink) {
        const uint32_t ds[4] = {r.d.x, r.d.y, r.d.z, r.d.w};
        const __nv_bfloat162 off = __float2bfloat162_rn(136.0f), zero = __float2bfloat162_rn(0.0f);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            sink.begin(a, 1);
#pragma unroll
            for (int bb = 0; bb < 2; ++bb) {
                const int b = 2 * a + bb;
                const uint4 q = r.q[b];
                const __nv_bfloat162 s = __float2bfloat162_rn(half_bits_to_float((ds[b >> 1] >> (16 * (b & 1))) & 0xffff));
                uint4 o;
                affine4(q.x & 0x0f0f0f0fu, off, s, zero, o.x, o.y); affine4(q.y & 0x0f0f0f0fu, off, s, zero, o.z, o.w);
                sink.emit(4 * b, o);
                affine4(q.z & 0x0f0f0f0fu, off, s, zero, o.x, o.y); affine4(q.w & 0x0f0f0f0fu, off, s, zero, o.z, o.w);
                sink.emit(4 * b + 1, o);
                affine4((q.x >> 4) & 0x0f0f0f0fu, off, s, zero, o.x, o.y); affine4((q.y >> 4) & 0x0f0f0f0fu, off, s, zero, o.z, o.w);
                sink.emit(4 * b + 2, o);
                affine4((q.z >> 4) & 0x0f0f0f0fu, off, s, zero, o.x, o.y); affine4((q.w >> 4) & 0x0f0f0f0fu, off, s, zero, o.z, o.w);
                sink.emit(4 * b + 3, o);
            }
            sink.end(a, 1);
        }
    }
};

template <> struct DequantBlock<FMT_IQ3_S> {
    struct Regs { uint2 qh; uint32_t sc; uint32_t d; uint4 sg[2]; uint4 qs[4]; };
    LLM_DEVICE static Regs load(const uint8_t* chunk, int g, int lane) {
        using T = FmtTraits<FMT_IQ3_S>;
        const int row = g * 32 + lane;
        Regs r;
        r.qh = ldg_nc_v2(chunk + T::P_QH + (row << 3));
        r.sc = ldg_nc_u32(chunk + T::P_SC + (row << 2));
        r.d = ldg_nc_u16(chunk + T::P_D + (row << 1));
        r.sg[0] = ldg_nc_v4(unit_ptr(chunk + T::P_SIGNS, 2, g, 0, lane));
        r.sg[1] = ldg_nc_v4(unit_ptr(chunk + T::P_SIGNS, 2, g, 1, lane));
#pragma unroll
        for (int u = 0; u < 4; ++u) r.qs[u] = ldg_nc_v4(unit_ptr(chunk + T::P_QS, 4, g, u, lane));
        return r;
    }
    // `grid`: the 512-entry codebook (shared or global memory).
    template <class S> LLM_DEVICE static void process(const Regs& r, S& sink, const uint32_t* grid) {
        const float d = half_bits_to_float((uint16_t)r.d);
        const __nv_bfloat162 off = __float2bfloat162_rn(128.0f), zero = __float2bfloat162_rn(0.0f);
#pragma unroll
        for (int ib = 0; ib < 8; ++ib) {
            if ((ib & 1) == 0) sink.begin(ib >> 1, 1);
            const uint4 q4 = r.qs[ib >> 1];
            const uint32_t qa = (ib & 1) ? q4.z : q4.x, qb = (ib & 1) ? q4.w : q4.y;
            const uint32_t hb = ((ib < 4 ? r.qh.x : r.qh.y) >> (8 * (ib & 3))) & 0xff;
            const uint4 s4 = r.sg[ib >> 2];
            const uint32_t sw = (ib & 3) == 0 ? s4.x : (ib & 3) == 1 ? s4.y : (ib & 3) == 2 ? s4.z : s4.w;
            const __nv_bfloat162 db = __float2bfloat162_rn(d * (1 + 2 * ((r.sc >> (4 * ib)) & 0xf)));
#pragma unroll
            for (int l = 0; l < 4; ++l) {
                const uint32_t pair = (l < 2 ? qa : qb) >> (16 * (l & 1));
                const uint32_t i1 = (pair & 0xff) | ((hb << (8 - 2 * l)) & 256);
                const uint32_t i2 = ((pair >> 8) & 0xff) | ((hb << (7 - 2 * l)) & 256);
                const uint32_t sb = (sw >> (8 * l)) & 0xff;
                uint4 o;
                affine4(grid[i1], off, db, zero, o.x, o.y);
                affine4(grid[i2], off, db, zero, o.z, o.w);
                o.x ^= ((sb & 1) << 15) | ((sb & 2) << 30);          // sign bit k of sb flips element k
                o.y ^= ((sb & 4) << 13) | ((sb & 8) << 28);
                o.z ^= ((sb & 16) << 11) | ((sb & 32) << 26);
                o.w ^= ((sb & 64) << 9) | ((sb & 128) << 24);
                sink.emit(4 * ib + l, o);
            }
            if (ib & 1) sink.end(ib >> 1, 1);
        }
    }
};

// Convenience: load + process in one go (no atom hooks needed).
template <int F, class S> LLM_DEVICE void dequant_block(const uint8_t* chunk, int g, int lane, S& sink) {
    const auto regs = DequantBlock<F>::load(chunk, g, lane);
    if constexpr (F == FMT_IQ3_S) DequantBlock<F>::process(regs, sink, g_iq3s_grid);
    else DequantBlock<F>::process(regs, sink);
}

}  // namespace llm
