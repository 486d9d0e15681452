// Mixture-of-experts routing for expert-parallel decode: RMSNorm + router projection + softmax + top-k (+ renormalise)
// + the grouped work list of the experts this rank owns, in one launch.
//
// One CTA per token.  The token's residual row is normalised into shared memory, the eight warps split the router rows
// (bf16 [experts, d], L2 resident), warp 0 takes softmax and the top-k (ties go to the lower expert id).  The CTA that
// finishes last (ticket) turns the [tokens, top_k] expert ids into work items: for every local expert the pairs routed
// to it, in token order, cut into groups of four.  The grouped GEMVs (gemv.cu, `GemvParams::items`) consume that list
// without a host round trip, so a decode step stays CUDA-graph capturable.
//
// Replaces the reference's route_logits / softmax_topk / count_per_expert / exclusive_scan / scatter_tokens kernels and the
// host-built expert lists between them (reference: src/v2/kernels/cuda/moe/CUDAMoEKernels.cu:66-700,
// src/v2/kernels/cuda/moe/CUDAMoEKernel.cpp).
#include "common.cuh"
#include "launch.h"
#include "gemv.h"

namespace llm {

constexpr int ROUTE_THREADS = 512;
constexpr int ROUTE_MAX_EXPERTS = 256;
constexpr int ROUTE_MAX_PAIRS = 4096;      // tokens * top_k handled by the list builder

__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_kernel(const MoeRouteParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float* xn = reinterpret_cast<float*>(smem_raw);                 // [d]
    float* logits = xn + p.d;                                        // [ROUTE_MAX_EXPERTS]
    __shared__ float s_part[ROUTE_THREADS / 32];
    pdl_trigger();
    pdl_wait();
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = blockIdx.x;

    // ---- RMSNorm of the token's row into shared memory ----
    const float* hrow = p.h + (size_t)t * p.h_stride;
    float ss = 0.f;
    for (int i = tid * 4; i < p.d; i += ROUTE_THREADS * 4) {
        const float4 v = *reinterpret_cast<const float4*>(hrow + i);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) s_part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < ROUTE_THREADS / 32; ++w) tot += s_part[w];
    const float rms = rsqrtf(tot / p.d + p.eps);
    for (int i = tid * 4; i < p.d; i += ROUTE_THREADS * 4) {
        const float4 v = *reinterpret_cast<const float4*>(hrow + i);
        const float4 g = *reinterpret_cast<const float4*>(p.norm_w + i);
        const float4 o = make_float4(v.x * rms * g.x, v.y * rms * g.y, v.z * rms * g.z, v.w * rms * g.w);
        *reinterpret_cast<float4*>(xn + i) = o;
        if (p.xn_out) *reinterpret_cast<uint2*>(p.xn_out + (size_t)t * p.d + i) = make_uint2(pack_bf16(o.x, o.y), pack_bf16(o.z, o.w));
    }
    __syncthreads();

    // ---- router projection: warp w takes experts w, w + 8, ...; eight experts at a time so that eight independent weight
    //      loads per lane are in flight for every read of the normalised row (a one-expert loop ran at memory latency:
    //      the expert weights of the layer before have flushed the router matrix out of L2 by the time it is needed) ----
    //      Every CTA walks the router rows from a different starting row: CTAs that read the same rows in lock step
    //      pile up on the same L2 slices.
    constexpr int NW = ROUTE_THREADS / 32, EB = 8;
    const int rot = (int)((blockIdx.x * 37u) % (unsigned)p.n_experts);
    for (int e0 = warp; e0 < p.n_experts; e0 += NW * EB) {
        const __nv_bfloat16* wrow[EB];
        float acc[EB];
        int eid[EB];
#pragma unroll
        for (int j = 0; j < EB; ++j) {
            const int e = e0 + j * NW;
            eid[j] = e < p.n_experts ? (e + rot) % p.n_experts : -1;
            wrow[j] = p.router + (size_t)(eid[j] < 0 ? 0 : eid[j]) * p.d;
            acc[j] = 0.f;
        }
#pragma unroll 2
        for (int i = lane * 4; i < p.d; i += 128) {            // consecutive lanes read consecutive 16 bytes of xn: no bank conflicts
            uint2 w4[EB];
#pragma unroll
            for (int j = 0; j < EB; ++j) w4[j] = *reinterpret_cast<const uint2*>(wrow[j] + i);
            const float4 a = *reinterpret_cast<const float4*>(xn + i);
#pragma unroll
            for (int j = 0; j < EB; ++j)
                acc[j] += bf16_lo(w4[j].x) * a.x + bf16_hi(w4[j].x) * a.y + bf16_lo(w4[j].y) * a.z + bf16_hi(w4[j].y) * a.w;
        }
#pragma unroll
        for (int j = 0; j < EB; ++j) {
            const float r = warp_sum(acc[j]);
            if (lane == 0 && eid[j] >= 0) logits[eid[j]] = r;
        }
    }
    __syncthreads();

    // ---- softmax over all experts, top-k with lower-id tie-break (warp 0) ----
    if (warp == 0) {
        constexpr int PER = ROUTE_MAX_EXPERTS / 32;
        float v[PER];
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = j * 32 + lane;
            v[j] = e < p.n_experts ? logits[e] : -INFINITY;
            mx = fmaxf(mx, v[j]);
        }
        mx = warp_max(mx);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            v[j] = (j * 32 + lane) < p.n_experts ? __expf(v[j] - mx) : -1.0f;
            sum += fmaxf(v[j], 0.f);
        }
        sum = warp_sum(sum);
        float wsum = 0.f, my_w = 0.f;
        int my_id = 0;
        for (int s = 0; s < p.top_k; ++s) {
            float best = -1.0f;
            int bi = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int e = j * 32 + lane;
                if (v[j] > best || (v[j] == best && e < bi)) { best = v[j]; bi = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
            }
            if ((bi & 31) == lane) v[bi >> 5] = -2.0f;
            const float pw = best / sum;
            wsum += pw;
            if (lane == s) { my_w = pw; my_id = bi; }
        }
        if (lane < p.top_k) {
            p.ids[(size_t)t * p.top_k + lane] = my_id;
            p.wts[(size_t)t * p.top_k + lane] = p.renorm ? my_w / wsum : my_w;
        }
    }
    if (p.items == nullptr) return;                                  // route-only call (prefill chunks): the caller groups on its own
    // ---- last CTA: build the grouped work list of the local experts ----
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(p.ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    int* s_ids = reinterpret_cast<int*>(smem_raw);                   // reuse: [pairs]
    __shared__ int s_cnt[ROUTE_MAX_EXPERTS], s_off[ROUTE_MAX_EXPERTS + 1];
    const int pairs = p.tokens * p.top_k;
    for (int i = tid; i < pairs; i += ROUTE_THREADS) s_ids[i] = __ldcg(p.ids + i);
    __syncthreads();
    // pass 1: pairs per local expert (warp w counts experts w, w + 8, ... with ballots over 32 pairs at a time)
    for (int el = warp; el < p.n_local; el += ROUTE_THREADS / 32) {
        const int e = p.e0 + el;
        int c = 0;
        for (int i0 = 0; i0 < pairs; i0 += 32) {
            const int i = i0 + lane;
            c += __popc(__ballot_sync(0xffffffffu, i < pairs && s_ids[i] == e));
        }
        if (lane == 0) {
            s_cnt[el] = c;
            if (p.counts) p.counts[el] = c;
        }
    }
    __syncthreads();
    // item offsets: exclusive scan of ceil(count / 4) by warp 0 (up to 8 experts per lane)
    if (warp == 0) {
        constexpr int PER = ROUTE_MAX_EXPERTS / 32;
        int loc[PER], sum = 0;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int el = lane * PER + j;
            loc[j] = el < p.n_local ? (s_cnt[el] + 3) >> 2 : 0;
            sum += loc[j];
        }
        int incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        int run = incl - sum;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int el = lane * PER + j;
            if (el < p.n_local) s_off[el] = run;
            run += loc[j];
        }
        const int total = __shfl_sync(0xffffffffu, incl, 31);
        if (lane == 0) {
            int n = total;
            if (n == 0) {                                            // keep the combine protocol alive on an idle rank
                p.items[0].expert = 0; p.items[0].m = 0;
                p.items[0].slot[0] = p.items[0].slot[1] = p.items[0].slot[2] = p.items[0].slot[3] = 0;
                n = 1;
            }
            *p.n_items = min(n, p.max_items);
            *p.ticket = 0u;
        }
    }
    __syncthreads();
    // pass 2: fill the items in token order; the pair of rank r within its expert goes to item off + r / 4, slot r % 4
    for (int el = warp; el < p.n_local; el += ROUTE_THREADS / 32) {
        const int cnt = s_cnt[el];
        if (cnt == 0) continue;
        const int e = p.e0 + el, off = s_off[el];
        int seen = 0;
        for (int i0 = 0; i0 < pairs && seen < cnt; i0 += 32) {
            const int i = i0 + lane;
            const bool hit = i < pairs && s_ids[i] == e;
            const unsigned mask = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int r = seen + __popc(mask & ((1u << lane) - 1u));
                const int item = off + (r >> 2);
                if (item < p.max_items) {
                    MoeItem& it = p.items[item];
                    it.slot[r & 3] = i;
                    if ((r & 3) == 0) { it.expert = el; it.m = min(4, cnt - r); }
                }
            }
            seen += __popc(mask);
        }
        __syncwarp();
        // pad the unused slots of the expert's last item with its first pair (rows are computed but never stored)
        const int last = off + ((cnt - 1) >> 2), used = ((cnt - 1) & 3) + 1;
        if (lane == 0 && last < p.max_items && used < 4) {
            __threadfence_block();
            MoeItem& it = p.items[last];
            const int first = it.slot[0];
            for (int m = used; m < 4; ++m) it.slot[m] = first;
        }
    }
}

// Weighted combine of the grouped expert outputs of a prefill chunk: h[t] += sum over the token's slots of wts[t, s] *
// y[pos[t, s]], where y holds the down-projection rows sorted by expert and pos is the inverse of that sort.  Slots with
// a zero weight (experts of another rank) are skipped.  One CTA per token; the slots are added in slot order, so the
// result does not depend on timing (reference: the ordered weighted scatter of its grouped prefill path,
// src/v2/kernels/cuda/moe/CUDAMoEKernels.cu:1826).
__global__ void __launch_bounds__(256) moe_combine_sorted_kernel(float* __restrict__ h, int h_stride, const float* __restrict__ y,
                                                                 const int* __restrict__ pos, const float* __restrict__ wts, int top_k, int d) {
    const int t = blockIdx.x;
    float* hrow = h + (size_t)t * h_stride;
    for (int i = threadIdx.x * 4; i < d; i += 256 * 4) {
        float4 acc = *reinterpret_cast<const float4*>(hrow + i);
        for (int s = 0; s < top_k; ++s) {
            const float w = wts[(size_t)t * top_k + s];
            if (w == 0.f) continue;
            const float4 v = *reinterpret_cast<const float4*>(y + (size_t)pos[(size_t)t * top_k + s] * d + i);
            acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
        }
        *reinterpret_cast<float4*>(hrow + i) = acc;
    }
}
cudaError_t launch_moe_combine_sorted(float* h, int h_stride, const float* y, const int* pos, const float* wts, int tokens, int top_k, int d,
                                      cudaStream_t st) {
    if (tokens == 0) return cudaSuccess;
    if (d % 4) return cudaErrorInvalidValue;
    moe_combine_sorted_kernel<<<tokens, 256, 0, st>>>(h, h_stride, y, pos, wts, top_k, d);
    return cudaGetLastError();
}

cudaError_t launch_moe_route(const MoeRouteParams& p, cudaStream_t st) {
    if (p.tokens == 0) return cudaSuccess;
    if (p.n_experts > ROUTE_MAX_EXPERTS || p.top_k > 32 || p.n_local > ROUTE_MAX_EXPERTS || (p.d & 255) != 0 ||
        (p.items != nullptr && p.tokens * p.top_k > ROUTE_MAX_PAIRS))
        return cudaErrorInvalidValue;
    const size_t dyn = max((size_t)(p.d + ROUTE_MAX_EXPERTS) * sizeof(float), p.items ? (size_t)p.tokens * p.top_k * sizeof(int) : (size_t)0);
    if (dyn > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
    return launch_pdl(moe_route_kernel, dim3(p.tokens), dim3(ROUTE_THREADS), dyn, st, p);
}

}  // namespace llm
