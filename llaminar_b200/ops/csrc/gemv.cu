// Small-batch (M <= 4 rows) GEMV straight from quantised weight chunks:  out[m, n] = sum_k x[m, k] * W[n, k].
//
// * lane == weight row: a warp owns 32 rows of a 128-row tile and walks 256-column chunks, so the
//   dot products need no cross-lane reduction and activations are shared-memory broadcasts;
// * activations are quantised to int8 per 32 columns in the kernel prologue (optionally after an
//   RMSNorm that is fused here too), weights are decoded in registers and multiplied with dp4a;
// * split-K over blockIdx.y with fp32 atomics into a scratch accumulator; the last CTA of a tile
//   applies the epilogue (bias / residual add / SwiGLU) and re-zeroes the scratch for the next call.
//
// Replaces the reference's nativeVnniGemv_* family + quantize_activations_blockwise_kernel +
// fused_swiglu_quantize_blockwise_kernel (reference: src/v2/kernels/cuda/gemm/CUDANativeVNNIGemvTuned.cu:332-1672,
// src/v2/kernels/cuda/ops/CUDAFusedOpsKernels.cu:37).
#include "formats.cuh"
#include "launch.h"
#include "gemv.h"
#include "tp_fuse.cuh"

namespace llm {

template <int M, int NORM>
LLM_DEVICE void gemv_prologue(const GemvParams& p, int kb0, int nkb, ActBlk* acts, float* s_red, const int (&xr)[M]) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float rms[M];
    if (NORM) {
        // full-row sum of squares (cheap: the row sits in L2), one value per activation row
        float ss[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            ss[m] = 0.f;
            const float4* x4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + (size_t)xr[m] * p.x_stride);
            for (int i = tid; i < p.k / 4; i += blockDim.x) {
                const float4 v = x4[i];
                ss[m] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            ss[m] = warp_sum(ss[m]);
            if (lane == 0) s_red[warp * M + m] = ss[m];
        }
        __syncthreads();
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float t = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_red[w * M + m];
            rms[m] = rsqrtf(t / p.k + p.eps);
        }
    }
    // quantise this CTA's column range: 4 consecutive columns per thread, 8 threads per 32-block
    const int n_quads = nkb * 64;
    for (int m = 0; m < M; ++m) {
        for (int qd = tid; qd < n_quads; qd += blockDim.x) {
            const int col = kb0 * 256 + qd * 4;
            float v0, v1, v2, v3;
            if (NORM) {
                const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + (size_t)xr[m] * p.x_stride + col);
                const float4 g = *reinterpret_cast<const float4*>(p.norm_w + col);
                v0 = v.x * rms[m] * g.x; v1 = v.y * rms[m] * g.y; v2 = v.z * rms[m] * g.z; v3 = v.w * rms[m] * g.w;
            } else {
                const uint2 v = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.x) + (size_t)xr[m] * p.x_stride + col);
                v0 = bf16_lo(v.x); v1 = bf16_hi(v.x); v2 = bf16_lo(v.y); v3 = bf16_hi(v.y);
            }
            float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float d = amax * (1.0f / 127.0f);
            const float inv = amax > 0.f ? 127.0f / amax : 0.f;
            const int q0 = __float2int_rn(v0 * inv), q1 = __float2int_rn(v1 * inv);
            const int q2 = __float2int_rn(v2 * inv), q3 = __float2int_rn(v3 * inv);
            int s = q0 + q1 + q2 + q3;
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            ActBlk& ab = acts[m * nkb + (qd >> 6)];
            const int qi = qd & 63;
            ab.a[qi] = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | ((q3 & 0xff) << 24);
            if ((qi & 7) == 0) ab.d[qi >> 3] = d;
            if ((qi & 3) == 0) ab.ds16[qi >> 2] = d * s;
        }
    }
    __syncthreads();
}

template <int FMT, int M, int NORM>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = blockIdx.x;
    const int per = (p.k_blocks + gridDim.y - 1) / gridDim.y;
    const int kb0 = blockIdx.y * per;
    const int kb1 = min(p.k_blocks, kb0 + per);
    const int nkb = max(kb1 - kb0, 0);
    // The weights do not depend on the previous kernel: pull this CTA's chunks towards L2 before waiting for it, so that
    // the HBM latency of the first loads overlaps the predecessor's tail and this kernel's activation prologue.
    if (!p.items && !p.expert_ids && nkb > 0) {
        const uint8_t* w0 = p.w + ((size_t)tile * p.k_blocks + kb0) * FmtTraits<FMT>::CHUNK;
        const int lines = min(nkb * (FmtTraits<FMT>::CHUNK / 128), 2048);          // at most 256 KB per CTA
        for (int i = tid; i < lines; i += 256) asm volatile("prefetch.global.L2 [%0];" ::"l"(w0 + (size_t)i * 128));
    }
    pdl_wait();
    // rows of this CTA: consecutive ones, or the (token, slot) pairs of a grouped-expert work item
    int xr[M], orow[M], n_valid = M, expert = -1;
    if (p.items) {
        if ((int)blockIdx.z >= __ldcg(p.n_items)) return;
        const MoeItem it = p.items[blockIdx.z];
        expert = it.expert;
        n_valid = min(it.m, M);
#pragma unroll
        for (int m = 0; m < M; ++m) { orow[m] = it.slot[m]; xr[m] = it.slot[m] / p.x_div; }
    } else {
#pragma unroll
        for (int m = 0; m < M; ++m) { orow[m] = blockIdx.z * M + m; xr[m] = (blockIdx.z / p.z_per_x) * M + m; }
        if (p.expert_ids) expert = p.expert_ids[blockIdx.z];
    }

    ActBlk* acts = reinterpret_cast<ActBlk*>(smem);
    float* s_red = reinterpret_cast<float*>(smem + (size_t)M * per * sizeof(ActBlk));   // [2][M][128] floats
    uint32_t* s_grid = reinterpret_cast<uint32_t*>(s_red + 2 * M * 128);
    if (FMT == FMT_IQ3_S) {
        for (int i = tid; i < 512; i += blockDim.x) s_grid[i] = g_iq3s_grid[i];
    }
    gemv_prologue<M, NORM>(p, kb0, nkb, acts, s_red, xr);

    const uint8_t* wbase = p.w;
    if (expert >= 0) wbase += (size_t)expert * p.expert_stride;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    const int g = warp & 3, kph = warp >> 2;
    const int act_stride = nkb * (int)sizeof(ActBlk);
    for (int kb = kb0 + kph; kb < kb1; kb += 2) {
        const uint8_t* chunk = wbase + ((size_t)tile * p.k_blocks + kb) * FmtTraits<FMT>::CHUNK;
        if constexpr (FMT == FMT_IQ3_S) DotBlock<FMT, M>::run(chunk, g, lane, acts + (kb - kb0), act_stride, acc, s_grid);
        else DotBlock<FMT, M>::run(chunk, g, lane, acts + (kb - kb0), act_stride, acc);
    }
    // combine the two k-phases
    const int r = g * 32 + lane;
#pragma unroll
    for (int m = 0; m < M; ++m) s_red[(kph * M + m) * 128 + r] = acc[m];
    __syncthreads();
    float v[M];
    if (tid < 128) {
#pragma unroll
        for (int m = 0; m < M; ++m) v[m] = s_red[m * 128 + tid] + s_red[(M + m) * 128 + tid];
    }
    const int row = tile * 128 + tid;
    if (gridDim.y > 1) {
        __shared__ int s_last;
        float* accum = p.accum + (size_t)blockIdx.z * M * p.accum_stride;
        if (tid < 128) {
#pragma unroll
            for (int m = 0; m < M; ++m) atomicAdd(&accum[(size_t)m * p.accum_stride + row], v[m]);
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned t = atomicAdd(&p.tickets[blockIdx.z * gridDim.x + tile], 1u);
            s_last = (t == gridDim.y - 1);
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        if (tid < 128) {
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float* a = &accum[(size_t)m * p.accum_stride + row];
                v[m] = __ldcg(a);
                __stcg(a, 0.f);
            }
        }
        if (tid == 0) p.tickets[blockIdx.z * gridDim.x + tile] = 0u;
    }
    // ---- epilogue ----
    if (p.epi == EPI_SWIGLU) {
        // a 32-row group holds 16 gate rows followed by the 16 matching up rows: pair lanes l and l + 16
        if (tid < 128) {
            const int col = tile * 64 + (tid >> 5) * 16 + (lane & 15);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float other = __shfl_xor_sync(0xffffffffu, v[m], 16);
                if (lane < 16 && col < p.n / 2 && m < n_valid)
                    static_cast<__nv_bfloat16*>(p.out)[(size_t)orow[m] * p.out_stride + col] = __float2bfloat16(silu(v[m]) * other);
            }
        }
        return;
    }
    if (p.epi == EPI_MOE_COMBINE) {
        // grouped expert down-projection: park this item's rows, and let the CTA that finishes the tile last do the
        // weighted combine over the locally owned pairs, the all-reduce across expert-parallel ranks and the residual add
        const MoeCombine& mc = p.moe;
        __shared__ int s_last2, s_ok2;
        __shared__ unsigned s_epoch2;
        if (tid < 128 && row < p.n) {
#pragma unroll
            for (int m = 0; m < M; ++m)
                if (m < n_valid) __stcg(&mc.yslot[(size_t)orow[m] * mc.y_stride + row], v[m]);
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned t = atomicAdd(&mc.tile_tickets[tile], 1u);
            s_last2 = (t == (unsigned)__ldcg(p.n_items) - 1u);
            if (s_last2 && p.tp) s_epoch2 = p.tp->epoch[tile];
        }
        __syncthreads();
        if (!s_last2) return;
        __threadfence();
        if (tid == 0) mc.tile_tickets[tile] = 0u;
        const int col = tile * 128 + (tid & 127), half = tid >> 7;
        const bool live = col < p.n;
        const TpFuse* tp = p.tp;
        const unsigned e = tp ? s_epoch2 : 0u;
        const int parity = e & 1;
        for (int t = half; t < mc.tokens; t += 2) {
            float sum = 0.f;
            if (live) {
                for (int j = 0; j < mc.top_k; ++j) {
                    const int pr = t * mc.top_k + j;
                    const int ex = mc.ids[pr] - mc.e0;
                    if ((unsigned)ex < (unsigned)mc.n_local) sum += mc.wts[pr] * __ldcg(&mc.yslot[(size_t)pr * mc.y_stride + col]);
                }
                if (!tp) {
                    mc.h[(size_t)t * mc.h_stride + col] += sum;
                } else {
                    for (int r = 0; r < tp->size; ++r)
                        tp->inbox[r][((size_t)(parity * tp->size + tp->rank) * tp->rows_cap + t) * tp->n_cap + col] = sum;
                }
            }
        }
        if (!tp) return;
        __syncthreads();
        if (tid < tp->size) tp_signal(*tp, tile, tid);
        if (tid == 0) {
            s_ok2 = tp_wait(*tp, tile, e) ? 1 : 0;
            tp->epoch[tile] = e + 1;
        }
        __syncthreads();
        if (!s_ok2 || !live) return;
        for (int t = half; t < mc.tokens; t += 2) {
            float sum = 0.f;
            for (int src = 0; src < tp->size; ++src)
                sum += __ldcg(tp->inbox[tp->rank] + ((size_t)(parity * tp->size + src) * tp->rows_cap + t) * tp->n_cap + col);
            mc.h[(size_t)t * mc.h_stride + col] += sum;
        }
        return;
    }
    if (p.tp != nullptr && p.epi == EPI_RESID) {
        // fused tensor-parallel all-reduce of this tile, then the residual add (see tp_fuse.cuh)
        __shared__ unsigned s_epoch;
        __shared__ int s_ok;
        const TpFuse& tp = *p.tp;
        if (tid == 0) s_epoch = tp.epoch[tile];
        __syncthreads();
        const unsigned e = s_epoch;
        auto row_of = [&](int i) { return orow[i]; };
        if (tid < 128 && row < p.n) {
            if (p.bias && tp.rank == 0) {
#pragma unroll
                for (int m = 0; m < M; ++m) v[m] += p.bias[row];
            }
            tp_push<M>(tp, e, row, v, row_of);
        }
        __syncthreads();
        if (tid < tp.size) tp_signal(tp, tile, tid);
        if (tid == 0) {
            s_ok = tp_wait(tp, tile, e) ? 1 : 0;
            tp.epoch[tile] = e + 1;
        }
        __syncthreads();
        if (s_ok && tid < 128 && row < p.n) {
            tp_reduce<M>(tp, e, row, v, row_of);
            float* h = static_cast<float*>(p.out);
#pragma unroll
            for (int m = 0; m < M; ++m) h[(size_t)orow[m] * p.out_stride + row] += v[m];
        }
        return;
    }
    if (tid < 128 && row < p.n) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m >= n_valid) break;
            float o = v[m];
            if (p.bias) o += p.bias[row];
            const size_t idx = (size_t)orow[m] * p.out_stride + row;
            if (p.epi == EPI_RESID) {
                float* h = static_cast<float*>(p.out);
                h[idx] = h[idx] + o;
            } else if (p.out_f32) {
                static_cast<float*>(p.out)[idx] = o;
            } else {
                static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16(o);
            }
        }
    }
}

template <int FMT, int M>
static cudaError_t launch_fm(const GemvParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    if (p.norm_w) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(gemv_kernel<FMT, M, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_pdl(gemv_kernel<FMT, M, 1>, grid, dim3(256), smem, st, p);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(gemv_kernel<FMT, M, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_pdl(gemv_kernel<FMT, M, 0>, grid, dim3(256), smem, st, p);
    }
    return cudaGetLastError();
}

template <int FMT>
static cudaError_t launch_f(const GemvParams& p, int mt, dim3 grid, size_t smem, cudaStream_t st) {
    switch (mt) {
        case 1: return launch_fm<FMT, 1>(p, grid, smem, st);
        case 2: return launch_fm<FMT, 2>(p, grid, smem, st);
        case 3: return launch_fm<FMT, 3>(p, grid, smem, st);
        case 4: return launch_fm<FMT, 4>(p, grid, smem, st);
    }
    return cudaErrorInvalidValue;
}

int gemv_pick_ksplit(int n_tiles, int k_blocks, int z) {
    // one full wave and no more: four CTAs fit an SM, and a second, mostly empty wave costs a whole CTA lifetime
    // (measured on 51200 x 5120: 400 CTAs 34.9 us, 800 CTAs 42.6 us); at least 2 chunks (one per k-phase) per CTA
    const int slots = 148 * 4;
    int ks = slots / (n_tiles * z);
    ks = ks < 1 ? 1 : ks;
    const int max_ks = k_blocks / 2 > 0 ? k_blocks / 2 : 1;
    return ks > max_ks ? max_ks : ks;
}

size_t gemv_smem_bytes(int m_tile, int k_blocks, int ksplit) {
    const int per = (k_blocks + ksplit - 1) / ksplit;
    return (size_t)m_tile * per * sizeof(ActBlk) + 2 * m_tile * 128 * sizeof(float) + 512 * sizeof(uint32_t);
}

// m_tile rows per CTA (1..4), z = number of row groups (grid.z); rows total = m_tile * z.
cudaError_t launch_gemv(const GemvParams& p, int m_tile, int z, cudaStream_t st) {
    if (m_tile < 1 || m_tile > 4 || z < 1) return cudaErrorInvalidValue;
    if (p.tp && z != 1 && p.epi != EPI_MOE_COMBINE) return cudaErrorInvalidValue;   // the per-tile flag protocol serves one row group
    if (p.items && (m_tile != 4 || !p.n_items || p.x_div < 1)) return cudaErrorInvalidValue;
    if (p.epi == EPI_MOE_COMBINE && (!p.items || !p.moe.yslot || !p.moe.tile_tickets)) return cudaErrorInvalidValue;
    int ks = p.ksplit > 0 ? p.ksplit : gemv_pick_ksplit(p.n_tiles, p.k_blocks, z);
    if (!p.accum || !p.tickets) ks = 1;
    size_t smem = gemv_smem_bytes(m_tile, p.k_blocks, ks);
    while (smem > 200 * 1024 && ks < p.k_blocks && p.accum) { ++ks; smem = gemv_smem_bytes(m_tile, p.k_blocks, ks); }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    dim3 grid(p.n_tiles, ks, z);
    switch (p.fmt) {
        case FMT_Q4_K: return launch_f<FMT_Q4_K>(p, m_tile, grid, smem, st);
        case FMT_Q5_K: return launch_f<FMT_Q5_K>(p, m_tile, grid, smem, st);
        case FMT_Q6_K: return launch_f<FMT_Q6_K>(p, m_tile, grid, smem, st);
        case FMT_Q8_0: return launch_f<FMT_Q8_0>(p, m_tile, grid, smem, st);
        case FMT_Q4_0: return launch_f<FMT_Q4_0>(p, m_tile, grid, smem, st);
        case FMT_IQ3_S: return launch_f<FMT_IQ3_S>(p, m_tile, grid, smem, st);
    }
    return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------------------------------
// dequantise chunks to a row-major bf16 matrix (debug / fallback) and gather-dequantise rows
// ------------------------------------------------------------------------------------------------
struct GlobalRowSink {
    __nv_bfloat16* dst;       // start of this row's 256-column block (nullptr: skip)
    LLM_DEVICE void begin(int, int) {}
    LLM_DEVICE void end(int, int) {}
    LLM_DEVICE void emit(int kg, uint4 v) { if (dst) *reinterpret_cast<uint4*>(dst + kg * 8) = v; }
};
struct GatherSink {
    float* f32; __nv_bfloat16* bf;
    LLM_DEVICE void begin(int, int) {}
    LLM_DEVICE void end(int, int) {}
    LLM_DEVICE void emit(int kg, uint4 v) {
        if (bf) *reinterpret_cast<uint4*>(bf + kg * 8) = v;
        if (f32) {
            *reinterpret_cast<float4*>(f32 + kg * 8) = make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
            *reinterpret_cast<float4*>(f32 + kg * 8 + 4) = make_float4(bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w));
        }
    }
};

template <int FMT>
__global__ void __launch_bounds__(128) dequant_kernel(const uint8_t* w, int n, int k, int k_blocks, __nv_bfloat16* out) {
    const int tile = blockIdx.x, kb = blockIdx.y, g = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint8_t* chunk = w + ((size_t)tile * k_blocks + kb) * FmtTraits<FMT>::CHUNK;
    const int row = tile * 128 + g * 32 + lane;
    GlobalRowSink sink{row < n ? out + (size_t)row * k + kb * 256 : nullptr};
    dequant_block<FMT>(chunk, g, lane, sink);
}

template <int FMT>
__global__ void __launch_bounds__(128) gather_rows_kernel(const uint8_t* w, int k_blocks, const int* rows, int n_rows,
                                                          float* out_f32, __nv_bfloat16* out_bf16, int out_stride) {
    pdl_trigger();
    pdl_wait();
    const int item = blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= n_rows * k_blocks) return;
    const int t = item / k_blocks, kb = item % k_blocks;
    const int r = rows[t];
    const int tile = r >> 7, g = (r >> 5) & 3, lane = r & 31;
    const uint8_t* chunk = w + ((size_t)tile * k_blocks + kb) * FmtTraits<FMT>::CHUNK;
    const size_t o = (size_t)t * out_stride + kb * 256;
    GatherSink sink{out_f32 ? out_f32 + o : nullptr, out_bf16 ? out_bf16 + o : nullptr};
    dequant_block<FMT>(chunk, g, lane, sink);
}

cudaError_t launch_dequant(int fmt, const uint8_t* w, int n, int k, __nv_bfloat16* out, cudaStream_t st) {
    const int nt = (n + 127) / 128, kb = k / 256;
    dim3 grid(nt, kb);
    switch (fmt) {
        case FMT_Q4_K: dequant_kernel<FMT_Q4_K><<<grid, 128, 0, st>>>(w, n, k, kb, out); break;
        case FMT_Q5_K: dequant_kernel<FMT_Q5_K><<<grid, 128, 0, st>>>(w, n, k, kb, out); break;
        case FMT_Q6_K: dequant_kernel<FMT_Q6_K><<<grid, 128, 0, st>>>(w, n, k, kb, out); break;
        case FMT_Q8_0: dequant_kernel<FMT_Q8_0><<<grid, 128, 0, st>>>(w, n, k, kb, out); break;
        case FMT_Q4_0: dequant_kernel<FMT_Q4_0><<<grid, 128, 0, st>>>(w, n, k, kb, out); break;
        case FMT_IQ3_S: dequant_kernel<FMT_IQ3_S><<<grid, 128, 0, st>>>(w, n, k, kb, out); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_gather_rows(int fmt, const uint8_t* w, int k, const int* rows, int n_rows, float* out_f32,
                               __nv_bfloat16* out_bf16, int out_stride, cudaStream_t st) {
    const int kb = k / 256;
    const int items = n_rows * kb;
    const int grid = (items + 127) / 128;
    if (grid == 0) return cudaSuccess;
    switch (fmt) {
        case FMT_Q4_K: return launch_pdl(gather_rows_kernel<FMT_Q4_K>, dim3(grid), dim3(128), 0, st, w, kb, rows, n_rows, out_f32, out_bf16, out_stride);
        case FMT_Q5_K: return launch_pdl(gather_rows_kernel<FMT_Q5_K>, dim3(grid), dim3(128), 0, st, w, kb, rows, n_rows, out_f32, out_bf16, out_stride);
        case FMT_Q6_K: return launch_pdl(gather_rows_kernel<FMT_Q6_K>, dim3(grid), dim3(128), 0, st, w, kb, rows, n_rows, out_f32, out_bf16, out_stride);
        case FMT_Q8_0: return launch_pdl(gather_rows_kernel<FMT_Q8_0>, dim3(grid), dim3(128), 0, st, w, kb, rows, n_rows, out_f32, out_bf16, out_stride);
        case FMT_Q4_0: return launch_pdl(gather_rows_kernel<FMT_Q4_0>, dim3(grid), dim3(128), 0, st, w, kb, rows, n_rows, out_f32, out_bf16, out_stride);
        case FMT_IQ3_S: return launch_pdl(gather_rows_kernel<FMT_IQ3_S>, dim3(grid), dim3(128), 0, st, w, kb, rows, n_rows, out_f32, out_bf16, out_stride);
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace llm
