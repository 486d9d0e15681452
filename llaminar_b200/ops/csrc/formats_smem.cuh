// Per-atom dequantisation of a weight chunk that has been staged in shared memory.
//
// A chunk (128 rows x 256 columns) splits into four 64-column "atoms", the K extent of one swizzled
// MMA operand tile.  DequantAtom<FMT, A>::run converts atom A of one row (lane == row inside the
// 32-row group g) to bf16 and hands it to the sink as eight 16-byte groups of 8 consecutive columns:
//     sink.emit(c, v)   c = 0..7 -> columns 64*A + 8*c .. + 7
// `raw` is the shared-memory address of the chunk; plane offsets are those of FmtTraits.
#pragma once
#include "formats.cuh"

namespace llm {

LLM_DEVICE uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
LLM_DEVICE uint2 lds_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
LLM_DEVICE uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
LLM_DEVICE uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
LLM_DEVICE uint32_t unit_off(int plane, int U, int g, int u, int lane) { return plane + ((((g * U + u) << 5) + lane) << 4); }

template <int F, int A> struct DequantAtom;

template <int A> struct DequantAtom<FMT_Q4_K, A> {
    template <class S> LLM_DEVICE static void run(uint32_t raw, int g, int lane, S& sink) {
        using T = FmtTraits<FMT_Q4_K>;
        const uint4 meta = lds_v4(raw + T::P_META + (((g << 5) + lane) << 4));
        const uint4 q0 = lds_v4(raw + unit_off(T::P_QS, 8, g, 2 * A, lane));
        const uint4 q1 = lds_v4(raw + unit_off(T::P_QS, 8, g, 2 * A + 1, lane));
        const float d = half_bits_to_float(meta.x & 0xffff), dmin = half_bits_to_float(meta.x >> 16);
        int sc[8], mn[8];
        unpack_k4_scales(meta.y, meta.z, meta.w, sc, mn);
        const __nv_bfloat162 off = __float2bfloat162_rn(128.0f);
        const __nv_bfloat162 s_lo = __float2bfloat162_rn(d * sc[2 * A]), b_lo = __float2bfloat162_rn(-dmin * mn[2 * A]);
        const __nv_bfloat162 s_hi = __float2bfloat162_rn(d * sc[2 * A + 1]), b_hi = __float2bfloat162_rn(-dmin * mn[2 * A + 1]);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 q = h ? q1 : q0;
            uint4 o;
            affine4(q.x & 0x0f0f0f0fu, off, s_lo, b_lo, o.x, o.y); affine4(q.y & 0x0f0f0f0fu, off, s_lo, b_lo, o.z, o.w);
            sink.emit(2 * h, o);
            affine4(q.z & 0x0f0f0f0fu, off, s_lo, b_lo, o.x, o.y); affine4(q.w & 0x0f0f0f0fu, off, s_lo, b_lo, o.z, o.w);
            sink.emit(2 * h + 1, o);
            affine4((q.x >> 4) & 0x0f0f0f0fu, off, s_hi, b_hi, o.x, o.y); affine4((q.y >> 4) & 0x0f0f0f0fu, off, s_hi, b_hi, o.z, o.w);
            sink.emit(4 + 2 * h, o);
            affine4((q.z >> 4) & 0x0f0f0f0fu, off, s_hi, b_hi, o.x, o.y); affine4((q.w >> 4) & 0x0f0f0f0fu, off, s_hi, b_hi, o.z, o.w);
            sink.emit(4 + 2 * h + 1, o);
        }
    }
};

template <int A> struct DequantAtom<FMT_Q5_K, A> {
    template <class S> LLM_DEVICE static void run(uint32_t raw, int g, int lane, S& sink) {
        using T = FmtTraits<FMT_Q5_K>;
        const uint4 meta = lds_v4(raw + T::P_META + (((g << 5) + lane) << 4));
        const float d = half_bits_to_float(meta.x & 0xffff), dmin = half_bits_to_float(meta.x >> 16);
        int sc[8], mn[8];
        unpack_k4_scales(meta.y, meta.z, meta.w, sc, mn);
        const __nv_bfloat162 off = __float2bfloat162_rn(128.0f);
        const __nv_bfloat162 s_lo = __float2bfloat162_rn(d * sc[2 * A]), b_lo = __float2bfloat162_rn(-dmin * mn[2 * A]);
        const __nv_bfloat162 s_hi = __float2bfloat162_rn(d * sc[2 * A + 1]), b_hi = __float2bfloat162_rn(-dmin * mn[2 * A + 1]);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 q = lds_v4(raw + unit_off(T::P_QS, 8, g, 2 * A + h, lane));
            const uint4 hq = lds_v4(raw + unit_off(T::P_QH, 2, g, h, lane));
            const uint32_t ws[4] = {q.x, q.y, q.z, q.w}, hs[4] = {hq.x, hq.y, hq.z, hq.w};
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                lo[i] = (ws[i] & 0x0f0f0f0fu) | (((hs[i] >> (2 * A)) & 0x01010101u) << 4);
                hi[i] = ((ws[i] >> 4) & 0x0f0f0f0fu) | (((hs[i] >> (2 * A + 1)) & 0x01010101u) << 4);
            }
            uint4 o;
            affine4(lo[0], off, s_lo, b_lo, o.x, o.y); affine4(lo[1], off, s_lo, b_lo, o.z, o.w);
            sink.emit(2 * h, o);
            affine4(lo[2], off, s_lo, b_lo, o.x, o.y); affine4(lo[3], off, s_lo, b_lo, o.z, o.w);
            sink.emit(2 * h + 1, o);
            affine4(hi[0], off, s_hi, b_hi, o.x, o.y); affine4(hi[1], off, s_hi, b_hi, o.z, o.w);
            sink.emit(4 + 2 * h, o);
            affine4(hi[2], off, s_hi, b_hi, o.x, o.y); affine4(hi[3], off, s_hi, b_hi, o.z, o.w);
            sink.emit(4 + 2 * h + 1, o);
        }
    }
};

template <int A> struct DequantAtom<FMT_Q6_K, A> {
    template <class S> LLM_DEVICE static void run(uint32_t raw, int g, int lane, S& sink) {
        using T = FmtTraits<FMT_Q6_K>;
        constexpr int n = A >> 1, hi_half = A & 1;           // atom 2n: low nibbles, atom 2n+1: high nibbles
        const int row = (g << 5) + lane;
        const uint4 scw = lds_v4(raw + T::P_SC + (row << 4));
        const uint32_t scs[4] = {scw.x, scw.y, scw.z, scw.w};
        const float d = half_bits_to_float((uint16_t)lds_u16(raw + T::P_D + (row << 1)));
        const __nv_bfloat162 off = __float2bfloat162_rn(160.0f), zero = __float2bfloat162_rn(0.0f);
#pragma unroll
        for (int lh = 0; lh < 2; ++lh) {
            const uint4 QA = lds_v4(raw + unit_off(T::P_QL, 8, g, 4 * n + lh, lane));
            const uint4 QB = lds_v4(raw + unit_off(T::P_QL, 8, g, 4 * n + 2 + lh, lane));
            const uint4 H = lds_v4(raw + unit_off(T::P_QH, 4, g, 2 * n + lh, lane));
            const uint32_t as_[4] = {QA.x, QA.y, QA.z, QA.w}, bs_[4] = {QB.x, QB.y, QB.z, QB.w}, hs_[4] = {H.x, H.y, H.z, H.w};
            constexpr int t0 = 2 * hi_half;                  // sub-block pair handled by this atom: t0, t0 + 1
            const int s0 = 8 * n + lh + 2 * t0, s1 = s0 + 2;
            const __nv_bfloat162 f0 = __float2bfloat162_rn(d * static_cast<int8_t>((scs[s0 >> 2] >> (8 * (s0 & 3))) & 0xff));
            const __nv_bfloat162 f1 = __float2bfloat162_rn(d * static_cast<int8_t>((scs[s1 >> 2] >> (8 * (s1 & 3))) & 0xff));
            uint32_t qa[4], qb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (hi_half == 0) {
                    qa[i] = (as_[i] & 0x0f0f0f0fu) | ((hs_[i] << 4) & 0x30303030u);
                    qb[i] = (bs_[i] & 0x0f0f0f0fu) | ((hs_[i] << 2) & 0x30303030u);
                } else {
                    qa[i] = ((as_[i] >> 4) & 0x0f0f0f0fu) | (hs_[i] & 0x30303030u);
                    qb[i] = ((bs_[i] >> 4) & 0x0f0f0f0fu) | ((hs_[i] >> 2) & 0x30303030u);
                }
            }
            uint4 o;
            affine4(qa[0], off, f0, zero, o.x, o.y); affine4(qa[1], off, f0, zero, o.z, o.w);
            sink.emit(2 * lh, o);
            affine4(qa[2], off, f0, zero, o.x, o.y); affine4(qa[3], off, f0, zero, o.z, o.w);
            sink.emit(2 * lh + 1, o);
            affine4(qb[0], off, f1, zero, o.x, o.y); affine4(qb[1], off, f1, zero, o.z, o.w);
            sink.emit(4 + 2 * lh, o);
            affine4(qb[2], off, f1, zero, o.x, o.y); affine4(qb[3], off, f1, zero, o.z, o.w);
            sink.emit(4 + 2 * lh + 1, o);
        }
    }
};

template <int A> struct DequantAtom<FMT_Q8_0, A> {
    template <class S> LLM_DEVICE static void run(uint32_t raw, int g, int lane, S& sink) {
        using T = FmtTraits<FMT_Q8_0>;
        const uint4 dw = lds_v4(raw + T::P_D + (((g << 5) + lane) << 4));
        const uint32_t ds[4] = {dw.x, dw.y, dw.z, dw.w};
#pragma unroll
        for (int uu = 0; uu < 4; ++uu) {
            const int u = 4 * A + uu, b = u >> 1;
            const uint4 q = lds_v4(raw + unit_off(T::P_QS, 16, g, u, lane));
            const float d = half_bits_to_float((ds[b >> 1] >> (16 * (b & 1))) & 0xffff);
            const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float v0 = d * static_cast<int8_t>(ws[i] & 0xff), v1 = d * static_cast<int8_t>((ws[i] >> 8) & 0xff);
                const float v2 = d * static_cast<int8_t>((ws[i] >> 16) & 0xff), v3 = d * static_cast<int8_t>(ws[i] >> 24);
                o[2 * i] = pack_bf16(v0, v1);
                o[2 * i + 1] = pack_bf16(v2, v3);
            }
            sink.emit(2 * uu, make_uint4(o[0], o[1], o[2], o[3]));
            sink.emit(2 * uu + 1, make_uint4(o[4], o[5], o[6], o[7]));
        }
    }
};

template <int A> struct DequantAtom<FMT_Q4_0, A> {
    template <class S> LLM_DEVICE static void run(uint32_t raw, int g, int lane, S& sink) {
        using T = FmtTraits<FMT_Q4_0>;
        const uint4 dw = lds_v4(raw + T::P_D + (((g << 5) + lane) << 4));
        const uint32_t ds[4] = {dw.x, dw.y, dw.z, dw.w};
        const __nv_bfloat162 off = __float2bfloat162_rn(136.0f), zero = __float2bfloat162_rn(0.0f);
#pragma unroll
        for (int bb = 0; bb < 2; ++bb) {
            const int b = 2 * A + bb;
            const uint4 q = lds_v4(raw + unit_off(T::P_QS, 8, g, b, lane));
            const __nv_bfloat162 s = __float2bfloat162_rn(half_bits_to_float((ds[b >> 1] >> (16 * (b & 1))) & 0xffff));
            uint4 o;
            affine4(q.x & 0x0f0f0f0fu, off, s, zero, o.x, o.y); affine4(q.y & 0x0f0f0f0fu, off, s, zero, o.z, o.w);
            sink.emit(4 * bb, o);
            affine4(q.z & 0x0f0f0f0fu, off, s, zero, o.x, o.y); affine4(q.w & 0x0f0f0f0fu, off, s, zero, o.z, o.w);
            sink.emit(4 * bb + 1, o);
            affine4((q.x >> 4) & 0x0f0f0f0fu, off, s, zero, o.x, o.y); affine4((q.y >> 4) & 0x0f0f0f0fu, off, s, zero, o.z, o.w);
            sink.emit(4 * bb + 2, o);
            affine4((q.z >> 4) & 0x0f0f0f0fu, off, s, zero, o.x, o.y); affine4((q.w >> 4) & 0x0f0f0f0fu, off, s, zero, o.z, o.w);
            sink.emit(4 * bb + 3, o);
        }
    }
};

template <int A> struct DequantAtom<FMT_IQ3_S, A> {
    // `grid`: shared-memory copy of the 512-entry codebook
    template <class S> LLM_DEVICE static void run(uint32_t raw, int g, int lane, S& sink, const uint32_t* grid) {
        using T = FmtTraits<FMT_IQ3_S>;
        const int row = (g << 5) + lane;
        const uint2 qh = lds_v2(raw + T::P_QH + (row << 3));
        const uint32_t scw = lds_u32(raw + T::P_SC + (row << 2));
        const float d = half_bits_to_float((uint16_t)lds_u16(raw + T::P_D + (row << 1)));
        const uint4 q4 = lds_v4(raw + unit_off(T::P_QS, 4, g, A, lane));
        const uint4 s4 = lds_v4(raw + unit_off(T::P_SIGNS, 2, g, A >> 1, lane));
        const __nv_bfloat162 off = __float2bfloat162_rn(128.0f), zero = __float2bfloat162_rn(0.0f);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            constexpr int dummy = 0; (void)dummy;
            const int ib = 2 * A + k;
            const uint32_t qa = k ? q4.z : q4.x, qb = k ? q4.w : q4.y;
            const uint32_t hb = ((ib < 4 ? qh.x : qh.y) >> (8 * (ib & 3))) & 0xff;
            const uint32_t sw = (ib & 3) == 0 ? s4.x : (ib & 3) == 1 ? s4.y : (ib & 3) == 2 ? s4.z : s4.w;
            const __nv_bfloat162 db = __float2bfloat162_rn(d * (1 + 2 * ((scw >> (4 * ib)) & 0xf)));
#pragma unroll
            for (int l = 0; l < 4; ++l) {
                const uint32_t pair = (l < 2 ? qa : qb) >> (16 * (l & 1));
                const uint32_t i1 = (pair & 0xff) | ((hb << (8 - 2 * l)) & 256);
                const uint32_t i2 = ((pair >> 8) & 0xff) | ((hb << (7 - 2 * l)) & 256);
                const uint32_t sb = (sw >> (8 * l)) & 0xff;
                uint4 o;
                affine4(grid[i1], off, db, zero, o.x, o.y);
                affine4(grid[i2], off, db, zero, o.z, o.w);
                o.x ^= ((sb & 1) << 15) | ((sb & 2) << 30);
                o.y ^= ((sb & 4) << 13) | ((sb & 8) << 28);
                o.z ^= ((sb & 16) << 11) | ((sb & 32) << 26);
                o.w ^= ((sb & 64) << 9) | ((sb & 128) << 24);
                sink.emit(4 * k + l, o);
            }
        }
    }
};

// ---- Q4_K to bf16, atom index at run time ------------------------------------------------------------------------------
// A nibble q kept in the high half of its byte (0xq0) and widened to 16 bits with a zero high byte is the bf16 subnormal
// 16 q * 2^-133 = q * 2^-129, exactly and with no magic offset to subtract afterwards.  One HFMA2 with the block's scale
// times 2^129 and its (negated) minimum then yields two weights with a single rounding: bit for bit what
// (128 + q - 128) * scale - min gives, for one half2 operation less per pair.  Per 8 weights: 3 logic ops, 4 byte permutes,
// 4 HFMA2 (the generic path spends 3 + 4 + 8).  The scale times 2^129 must stay finite in bf16, i.e. d * sc < 0.5 (weights
// up to about +-7); larger scales are clamped to the largest finite value, and the loader re-encodes such a tensor instead
// of sending it here (ops/layout.py: q4k_scales_in_range).
// The atom index is a run-time value so that the four warps of a scheduler (same row group, different atoms) share one
// copy of the code.  The sink receives the whole atom at once: sink.emit64(r) -> the 64 columns of atom A of this lane's row.
// (A fp16 variant through cvt.rn.f16x2.e4m3x2 was tried first: tcgen05.mma kind::f16 with an fp16 A and a bf16 B operand
// raises "illegal instruction" on B200, although the two formats are separate fields of the instruction descriptor.)
LLM_DEVICE uint32_t hfma2_bf16_u32(uint32_t a, __nv_bfloat162 s, __nv_bfloat162 b) {
    const __nv_bfloat162 r = __hfma2(*reinterpret_cast<const __nv_bfloat162*>(&a), s, b);
    return *reinterpret_cast<const uint32_t*>(&r);
}
struct DequantAtomQ4KRt {
    template <bool HI>
    LLM_DEVICE static void conv16(const uint4& q, __nv_bfloat162 s, __nv_bfloat162 nb, uint32_t* r) {
        const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = (HI ? ws[i] : (ws[i] << 4)) & 0xf0f0f0f0u;
            r[2 * i] = hfma2_bf16_u32(__byte_perm(w, 0u, 0x4140), s, nb);
            r[2 * i + 1] = hfma2_bf16_u32(__byte_perm(w, 0u, 0x4342), s, nb);
        }
    }
    // Everything this thread needs from the raw chunk, fetched and prepared before the operand slot is waited for: the two
    // 16-byte units of packed nibbles and the scale / minimum pairs of sub-blocks 2A and 2A + 1.
    struct Regs { uint4 q0, q1; __nv_bfloat162 s_lo, s_hi, b_lo, b_hi; };
    LLM_DEVICE static Regs load(uint32_t raw, int g, int lane, int A) {
        using T = FmtTraits<FMT_Q4_K>;
        Regs r;
        const uint32_t row16 = (uint32_t)((g << 5) + lane) << 4;
        const uint4 meta = lds_v4(raw + T::P_META + row16);
        const uint32_t qaddr = raw + T::P_QS + ((uint32_t)(g * 8 + 2 * A) << 9) + ((uint32_t)lane << 4);
        r.q0 = lds_v4(qaddr);
        r.q1 = lds_v4(qaddr + 512);
        // 6-bit scales / minima of sub-blocks 2A and 2A + 1: bytes (2A & 3) and (2A & 3) + 1 of the three packed words
        const int sh = (A & 1) << 4;
        const uint32_t a2 = meta.y >> sh, b2 = meta.z >> sh, c2 = meta.w >> sh;
        uint32_t sc2, mn2;
        if (A < 2) { sc2 = a2 & 0x3f3fu; mn2 = b2 & 0x3f3fu; }
        else { sc2 = (c2 & 0x0f0fu) | ((a2 >> 2) & 0x3030u); mn2 = ((c2 >> 4) & 0x0f0fu) | ((b2 >> 2) & 0x3030u); }
        // d * 2^129 in two exact steps (2^129 is not an fp32 value).  The 6-bit integers become floats without the conversion
        // unit: byte k under the exponent of 2^23 is 2^23 + k, and (2^23 + k) * f - 2^23 * f is one FMA.
        const float BIG = 3.3895314e38f;                       // largest finite bf16
        const float d100 = half_bits_to_float(meta.x & 0xffff) * 1.2676506e30f;     // d * 2^100
        const float ndmin = -half_bits_to_float(meta.x >> 16);
        const float d100c = -8388608.0f * d100, ndminc = -8388608.0f * ndmin;
        const float k29 = 536870912.0f;                         // 2^29
        const float sc_lo = __uint_as_float(__byte_perm(sc2, 0x4b000000u, 0x7650)), sc_hi = __uint_as_float(__byte_perm(sc2, 0x4b000000u, 0x7651));
        const float mn_lo = __uint_as_float(__byte_perm(mn2, 0x4b000000u, 0x7650)), mn_hi = __uint_as_float(__byte_perm(mn2, 0x4b000000u, 0x7651));
        r.s_lo = __float2bfloat162_rn(fminf(fmaf(sc_lo, d100, d100c) * k29, BIG));
        r.s_hi = __float2bfloat162_rn(fminf(fmaf(sc_hi, d100, d100c) * k29, BIG));
        r.b_lo = __float2bfloat162_rn(fmaf(mn_lo, ndmin, ndminc));
        r.b_hi = __float2bfloat162_rn(fmaf(mn_hi, ndmin, ndminc));
        return r;
    }
    // all 64 values (32 packed pairs) of the atom into `o`, which the caller then hands to one tensor-memory store
    LLM_DEVICE static void convert(const Regs& r, uint32_t (&o)[32]) {
        conv16<false>(r.q0, r.s_lo, r.b_lo, o);
        conv16<false>(r.q1, r.s_lo, r.b_lo, o + 8);
        conv16<true>(r.q0, r.s_hi, r.b_hi, o + 16);
        conv16<true>(r.q1, r.s_hi, r.b_hi, o + 24);
    }
};

}  // namespace llm
