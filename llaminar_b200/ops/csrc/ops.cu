// Memory-bound glue kernels: RMSNorm, fused QK-norm + RoPE + paged KV append, SwiGLU, sampling
// (argmax, top-k/top-p, penalties), speculative-decode verification, MoE routing, NaN/Inf scan.
// Reference counterparts: src/v2/kernels/cuda/ops/CUDARMSNormKernels.cu, CUDARoPEKernels.cu,
// CUDAFusedOpsKernels.cu, CUDASamplingKernels.cu, src/v2/kernels/cuda/kvcache/CUDARingKVCache.cu
// (ring append; here the cache is paged), src/v2/kernels/cuda/moe/CUDAMoEKernels.cu (softmax_topk),
// src/v2/backends/cuda/CUDATensorValidation.cu.
#include "common.cuh"
#include "launch.h"
#include "ops.h"

namespace llm {

constexpr int PAGE = 64;

// ------------------------------------------------------------------------------------------------
// RMSNorm: fp32 residual stream in, bf16 out
// ------------------------------------------------------------------------------------------------
// One CTA per row.  For rows of up to 8192 values the row and the gain are read once, together, and stay in registers across
// the reduction (one memory round trip on the critical path of a decode step instead of two); longer rows are re-read.
// `h` is written by the kernel before this one, which may still be running when this kernel's CTAs become resident
// (programmatic dependent launch): it is read with L2-coherent loads (`__ldcg`), never through the read-only path.
template <bool IN_REGS>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* h, const float* __restrict__ w,
                                                      __nv_bfloat16* __restrict__ out, int d, float eps) {
    __shared__ float s_part[8];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const float4* x4 = reinterpret_cast<const float4*>(h + (size_t)row * d);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    constexpr int MAXV = 8;
    float4 xv[MAXV], gv[MAXV];
    float ss = 0.f;
    if (IN_REGS) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int i = tid + j * 256;
            if (i < d / 4) { xv[j] = __ldcg(x4 + i); gv[j] = w4[i]; }
            else { xv[j] = make_float4(0.f, 0.f, 0.f, 0.f); gv[j] = xv[j]; }
        }
#pragma unroll
        for (int j = 0; j < MAXV; ++j) ss += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
    } else {
        for (int i = tid; i < d / 4; i += 256) {
            const float4 v = __ldcg(x4 + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) s_part[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_part[i];
    const float r = rsqrtf(tot / d + eps);
    uint2* o2 = reinterpret_cast<uint2*>(out + (size_t)row * d);
    if (IN_REGS) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int i = tid + j * 256;
            if (i < d / 4)
                o2[i] = make_uint2(pack_bf16(xv[j].x * r * gv[j].x, xv[j].y * r * gv[j].y), pack_bf16(xv[j].z * r * gv[j].z, xv[j].w * r * gv[j].w));
        }
    } else {
        for (int i = tid; i < d / 4; i += 256) {
            const float4 v = __ldcg(x4 + i), g = w4[i];
            o2[i] = make_uint2(pack_bf16(v.x * r * g.x, v.y * r * g.y), pack_bf16(v.z * r * g.z, v.w * r * g.w));
        }
    }
}

LLM_DEFINE_BOUNDS_STATUS_READER(bounds_status_ops)

cudaError_t launch_rmsnorm(const float* h, const float* w, __nv_bfloat16* out, int rows, int d, float eps, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    if (d % 4) return cudaErrorInvalidValue;
    if (d <= 8 * 256 * 4) return launch_pdl(rmsnorm_kernel<true>, dim3(rows), dim3(256), 0, st, h, w, out, d, eps);
    return launch_pdl(rmsnorm_kernel<false>, dim3(rows), dim3(256), 0, st, h, w, out, d, eps);
}

// ------------------------------------------------------------------------------------------------
// Owner side of the fused reduce-scatter (RsFuse, gemm_tc.h): one CTA per row this rank owns.  It waits (bounded) until every
// rank's partial tiles of the row's block have arrived, adds them in rank order to the fp32 residual row, writes the row back
// and, when a norm gain is given, the bf16 RMSNorm of the new row (the input of the next column-parallel projection, placed
// where the all-gather reads it).  Replaces the reference's all-reduce + residual add + RMSNorm stages
// (reference: src/v2/models/qwen/QwenGraphBase.cpp:2004-2023, :2937-3014).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rs_reduce_norm_kernel(const __nv_bfloat16* inbox, const unsigned* flags, unsigned target,
                                                             int world, int rows_per_rank, int n_cap, int block_m, float* __restrict__ h,
                                                             const float* __restrict__ norm_w, __nv_bfloat16* __restrict__ xn, int d, float eps,
                                                             unsigned spin_limit, int* status) {
    __shared__ float s_part[8];
    __shared__ int s_ok;
    const int row = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) {
        const unsigned* f = flags + row / block_m;
        int ok = 0;
        for (unsigned i = 0; i < spin_limit; ++i) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (v >= target) { ok = 1; break; }
            if (i > 1024) __nanosleep(100);
        }
        if (!ok && status) atomicExch(status, (int)STATUS_TIMEOUT);
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;                                   // the row keeps its old value; the host sees the status word
    constexpr int MAXU = 4;                              // 8-column units per thread: d <= 8192
    float acc[MAXU][8];
    float ss = 0.f;
    float* hrow = h + (size_t)row * d;
    const int units = d >> 3;
#pragma unroll
    for (int j = 0; j < MAXU; ++j) {
        const int u = tid + j * 256;
        if (u < units) {
            const float4 a = *reinterpret_cast<const float4*>(hrow + u * 8), b = *reinterpret_cast<const float4*>(hrow + u * 8 + 4);
            acc[j][0] = a.x; acc[j][1] = a.y; acc[j][2] = a.z; acc[j][3] = a.w;
            acc[j][4] = b.x; acc[j][5] = b.y; acc[j][6] = b.z; acc[j][7] = b.w;
            for (int src = 0; src < world; ++src) {
                const uint4 v = __ldcg(reinterpret_cast<const uint4*>(inbox + ((size_t)src * rows_per_rank + row) * n_cap + u * 8));
                acc[j][0] += bf16_lo(v.x); acc[j][1] += bf16_hi(v.x); acc[j][2] += bf16_lo(v.y); acc[j][3] += bf16_hi(v.y);
                acc[j][4] += bf16_lo(v.z); acc[j][5] += bf16_hi(v.z); acc[j][6] += bf16_lo(v.w); acc[j][7] += bf16_hi(v.w);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += acc[j][i] * acc[j][i];
            *reinterpret_cast<float4*>(hrow + u * 8) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
            *reinterpret_cast<float4*>(hrow + u * 8 + 4) = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
        }
    }
    if (norm_w == nullptr) return;
    ss = warp_sum(ss);
    if ((tid & 31) == 0) s_part[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_part[i];
    const float r = rsqrtf(tot / d + eps);
    __nv_bfloat16* xrow = xn + (size_t)row * d;
#pragma unroll
    for (int j = 0; j < MAXU; ++j) {
        const int u = tid + j * 256;
        if (u < units) {
            const float4 g0 = *reinterpret_cast<const float4*>(norm_w + u * 8), g1 = *reinterpret_cast<const float4*>(norm_w + u * 8 + 4);
            uint4 o;
            o.x = pack_bf16(acc[j][0] * r * g0.x, acc[j][1] * r * g0.y);
            o.y = pack_bf16(acc[j][2] * r * g0.z, acc[j][3] * r * g0.w);
            o.z = pack_bf16(acc[j][4] * r * g1.x, acc[j][5] * r * g1.y);
            o.w = pack_bf16(acc[j][6] * r * g1.z, acc[j][7] * r * g1.w);
            *reinterpret_cast<uint4*>(xrow + u * 8) = o;
        }
    }
}
cudaError_t launch_rs_reduce_norm(const __nv_bfloat16* inbox, const unsigned* flags, unsigned target, int world, int rows_per_rank, int n_cap,
                                  int block_m, float* h, const float* norm_w, __nv_bfloat16* xn, int rows, int d, float eps,
                                  unsigned spin_limit, int* status, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    if (d % 8 || d > 8192 || rows > rows_per_rank || block_m < 1) return cudaErrorInvalidValue;
    rs_reduce_norm_kernel<<<rows, 256, 0, st>>>(inbox, flags, target, world, rows_per_rank, n_cap, block_m, h, norm_w, xn, d, eps, spin_limit, status);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Multi-token-prediction draft prologue: out[row] = [RMSNorm(embedding[row]; enorm) | RMSNorm(hidden[row]; hnorm)] as bf16,
// the input of the NextN layer's eh_proj (reference: src/v2/kernels/cuda/ops/CUDARowSelectKernels.cu:74 mtpConcatFP32Kernel
// after two RMSNorm stages, src/v2/models/qwen35/Qwen35Graph.cpp:403-507).  grid = (rows, 2): y selects the half.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) mtp_concat_norm_kernel(const float* __restrict__ emb, const float* __restrict__ hidden,
                                                              const float* __restrict__ enorm, const float* __restrict__ hnorm,
                                                              __nv_bfloat16* __restrict__ out, int d, float eps) {
    __shared__ float s_part[8];
    const int row = blockIdx.x, half = blockIdx.y, tid = threadIdx.x;
    const float4* x4 = reinterpret_cast<const float4*>((half ? hidden : emb) + (size_t)row * d);
    const float4* w4 = reinterpret_cast<const float4*>(half ? hnorm : enorm);
    float ss = 0.f;
    for (int i = tid; i < d / 4; i += 256) {
        const float4 v = x4[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) s_part[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_part[i];
    const float r = rsqrtf(tot / d + eps);
    uint2* o2 = reinterpret_cast<uint2*>(out + (size_t)row * 2 * d + (size_t)half * d);
    for (int i = tid; i < d / 4; i += 256) {
        const float4 v = x4[i], g = w4[i];
        o2[i] = make_uint2(pack_bf16(v.x * r * g.x, v.y * r * g.y), pack_bf16(v.z * r * g.z, v.w * r * g.w));
    }
}
cudaError_t launch_mtp_concat_norm(const float* emb, const float* hidden, const float* enorm, const float* hnorm,
                                   __nv_bfloat16* out, int rows, int d, float eps, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    if (d % 4) return cudaErrorInvalidValue;
    mtp_concat_norm_kernel<<<dim3(rows, 2), 256, 0, st>>>(emb, hidden, enorm, hnorm, out, d, eps);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// per-head QK RMSNorm + split-half RoPE + paged KV append: one warp per (token, head)
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) rope_kv_kernel(const RopeKVParams p) {
    constexpr int EPL = D / 64;                          // elements per lane in each half
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int heads_total = p.n_heads + 2 * p.n_kv_heads;
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= p.n_tokens * heads_total) return;
    const int t = item / heads_total, hh = item % heads_total;
    const __nv_bfloat16* src = p.qkv + (size_t)t * heads_total * D + (size_t)hh * D;
    const int pos = p.positions[t];
    float a[EPL], b[EPL];                                // a: first half, b: second half
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        a[e] = __bfloat162float(src[lane * EPL + e]);
        b[e] = __bfloat162float(src[D / 2 + lane * EPL + e]);
    }
    const bool is_q = hh < p.n_heads, is_k = !is_q && hh < p.n_heads + p.n_kv_heads;
    if (is_q || is_k) {
        const float* nw = is_q ? p.q_norm : p.k_norm;
        if (nw) {
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) ss += a[e] * a[e] + b[e] * b[e];
            ss = warp_sum(ss);
            const float r = rsqrtf(ss / D + p.eps);
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                a[e] *= r * nw[lane * EPL + e];
                b[e] *= r * nw[D / 2 + lane * EPL + e];
            }
        }
        const float l2t = log2f(p.theta);
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            const int i = lane * EPL + e;
            const float inv = exp2f(-(2.0f * i / D) * l2t);
            float sn, cs;
            sincosf(pos * inv, &sn, &cs);
            const float x1 = a[e], x2 = b[e];
            a[e] = x1 * cs - x2 * sn;
            b[e] = x2 * cs + x1 * sn;
        }
    }
    __nv_bfloat16* dst;
    if (is_q) {
        dst = p.q_out + ((size_t)t * p.n_heads + hh) * D;
    } else {
        const int kvh = is_k ? hh - p.n_heads : hh - p.n_heads - p.n_kv_heads;
        const int seq = LLM_CHECK_INDEX(p.seq_ids[t], p.n_seqs);
        const int slot = LLM_CHECK_INDEX(pos / PAGE, p.max_pages);
        const size_t page = (size_t)LLM_CHECK_INDEX(p.block_table[(size_t)seq * p.max_pages + slot], p.n_pages);
        if (p.kv_q8) {
            // 8-bit cache: one fp16 scale per 32 values (amax / 127), values rounded to nearest.  This lane's values sit in
            // blocks (lane * EPL) / 32 of the first half and the same block of the second half; the lanes of a block are
            // 32 / EPL neighbours.
            constexpr int GROUP = 32 / EPL;
            float ma = 0.f, mb = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) { ma = fmaxf(ma, fabsf(a[e])); mb = fmaxf(mb, fabsf(b[e])); }
#pragma unroll
            for (int o = 1; o < GROUP; o <<= 1) {
                ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, o));
                mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, o));
            }
            // The stored scale is amax / 127 rounded UP to seven mantissa bits (no value clips; the values are quantised with
            // the stored scale).  Seven bits because the decode kernel expands a byte as (1152 + x) * s - 1152 * s in one fp16
            // FMA, and 1152 * s = 9 * s * 2^7 is exact in fp16 only if s carries at most seven bits.
            auto scale7 = [](float amax) {
                const uint32_t b = (__float_as_uint(amax * (1.0f / 127.0f)) + 0xFFFFu) & 0xFFFF0000u;
                return __uint_as_float(b);
            };
            const __half ha = __float2half_rn(scale7(ma)), hb = __float2half_rn(scale7(mb));
            const float da = __half2float(ha), db = __half2float(hb);
            const float ia = da > 0.f ? 1.0f / da : 0.f, ib = db > 0.f ? 1.0f / db : 0.f;
            uint8_t* pg = reinterpret_cast<uint8_t*>(p.kv) + page * p.page_bytes;
            const size_t row = ((size_t)(is_k ? 0 : 1) * p.n_kv_heads + kvh) * PAGE + (size_t)(pos % PAGE);
            int8_t* d8 = reinterpret_cast<int8_t*>(pg + row * D);
            __half* sc = reinterpret_cast<__half*>(pg + p.scale_off + row * (D / 32) * 2);
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                d8[lane * EPL + e] = (int8_t)max(-127, min(127, __float2int_rn(a[e] * ia)));
                d8[D / 2 + lane * EPL + e] = (int8_t)max(-127, min(127, __float2int_rn(b[e] * ib)));
            }
            if ((lane & (GROUP - 1)) == 0) {
                sc[(lane * EPL) / 32] = ha;
                sc[(D / 2 + lane * EPL) / 32] = hb;
            }
            return;
        }
        dst = p.kv + ((page * 2 + (is_k ? 0 : 1)) * p.n_kv_heads + kvh) * (size_t)(PAGE * D) + (size_t)(pos % PAGE) * D;
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        dst[lane * EPL + e] = __float2bfloat16(a[e]);
        dst[D / 2 + lane * EPL + e] = __float2bfloat16(b[e]);
    }
}

cudaError_t launch_rope_kv(const RopeKVParams& p, cudaStream_t st) {
    const int items = p.n_tokens * (p.n_heads + 2 * p.n_kv_heads);
    if (items == 0) return cudaSuccess;
    const int grid = (items + 3) / 4;
    if (p.head_dim == 128) return launch_pdl(rope_kv_kernel<128>, dim3(grid), dim3(128), 0, st, p);
    else if (p.head_dim == 64) return launch_pdl(rope_kv_kernel<64>, dim3(grid), dim3(128), 0, st, p);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// 8-bit KV pages -> bf16 pages (the prefill kernels read bf16): one CTA per (page slot, sequence), one 16-byte unit of
// 16 values per thread and step
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) kv_dequant_pages_kernel(const uint8_t* kv8, size_t page_bytes, size_t scale_off,
                                                               const int* block_table, const int* n_tokens, int max_pages,
                                                               int n_kv_heads, int head_dim, int n_pages, __nv_bfloat16* __restrict__ staging) {
    pdl_trigger();
    pdl_wait();
    const int j = blockIdx.x, s = blockIdx.y;
    if (j * PAGE >= n_tokens[s]) return;
    const size_t page = (size_t)LLM_CHECK_INDEX(block_table[(size_t)s * max_pages + j], n_pages);
    const uint8_t* pg = kv8 + page * page_bytes;
    const int rows = 2 * n_kv_heads * PAGE, upr = head_dim / 16;           // 16-value units per row
    __nv_bfloat16* out = staging + ((size_t)s * max_pages + j) * (size_t)rows * head_dim;
    for (int idx = threadIdx.x; idx < rows * upr; idx += blockDim.x) {
        const int row = idx / upr, u = idx - row * upr;
        const uint4 w = __ldcg(reinterpret_cast<const uint4*>(pg + (size_t)row * head_dim + u * 16));   // written by the kernel before (see rmsnorm_kernel)
        const float sc = __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(pg + scale_off + ((size_t)row * (head_dim / 32) + (u >> 1)) * 2))));
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int8_t b0 = (int8_t)(ws[k] & 0xff), b1 = (int8_t)((ws[k] >> 8) & 0xff), b2 = (int8_t)((ws[k] >> 16) & 0xff), b3 = (int8_t)(ws[k] >> 24);
            o[2 * k] = pack_bf16(sc * b0, sc * b1);
            o[2 * k + 1] = pack_bf16(sc * b2, sc * b3);
        }
        uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * head_dim + u * 16);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}
cudaError_t launch_kv_dequant_pages(const uint8_t* kv8, size_t page_bytes, size_t scale_off, const int* block_table, const int* n_tokens,
                                    int n_seqs, int max_pages, int n_kv_heads, int head_dim, int n_pages, __nv_bfloat16* staging, cudaStream_t st) {
    if (n_seqs == 0 || max_pages == 0) return cudaSuccess;
    if (head_dim % 32 != 0) return cudaErrorInvalidValue;
    return launch_pdl(kv_dequant_pages_kernel, dim3(max_pages, n_seqs), dim3(256), 0, st, kv8, page_bytes, scale_off, block_table, n_tokens,
                      max_pages, n_kv_heads, head_dim, n_pages, staging);
}

// ------------------------------------------------------------------------------------------------
// sampling
// ------------------------------------------------------------------------------------------------
LLM_DEVICE uint32_t order_key(float f) {                 // monotone float -> uint map
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
LLM_DEVICE float key_to_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
LLM_DEVICE uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
LLM_DEVICE float uniform01(uint64_t seed, uint64_t ctr) {
    return (splitmix64(seed ^ splitmix64(ctr)) >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(1024) argmax_kernel(const float* logits, int vocab, int stride, int* __restrict__ tokens,
                                                      int* __restrict__ pairs, int idx_offset) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    pdl_trigger();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * stride;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += 1024) {
        const float v = __ldcg(row + i);             // the head's output: L2-coherent load (see rmsnorm_kernel)
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = best; s_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = s_v[threadIdx.x]; bi = s_i[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) {
            bi = bi == 0x7fffffff ? 0 : bi;
            if (tokens) tokens[blockIdx.x] = bi;
            if (pairs) {                       // (value bits, global index) for the cross-rank merge of a vocabulary-sharded head
                pairs[2 * blockIdx.x] = __float_as_int(best);
                pairs[2 * blockIdx.x + 1] = bi + idx_offset;
            }
        }
    }
}
cudaError_t launch_argmax(const float* logits, int rows, int vocab, int stride, int* tokens, int* pairs, int idx_offset, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    return launch_pdl(argmax_kernel, dim3(rows), dim3(1024), 0, st, logits, vocab, stride, tokens, pairs, idx_offset);
}

// Merge of per-shard argmax candidates: gathered[rank][row] = (value bits, global index); larger value wins, ties go to
// the lower index (the result equals the argmax over the full row).
__global__ void argmax_merge_kernel(const int* __restrict__ gathered, int ranks, int rows, int* __restrict__ tokens) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int k = 0; k < ranks; ++k) {
        const float v = __int_as_float(gathered[((size_t)k * rows + r) * 2]);
        const int i = gathered[((size_t)k * rows + r) * 2 + 1];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    tokens[r] = bi == 0x7fffffff ? 0 : bi;
}
cudaError_t launch_argmax_merge(const int* gathered, int ranks, int rows, int* tokens, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    argmax_merge_kernel<<<(rows + 127) / 128, 128, 0, st>>>(gathered, ranks, rows, tokens);
    return cudaGetLastError();
}

// top-k (radix select) -> sort candidates -> softmax -> top-p cut -> inverse-CDF sample.  One CTA per row.
constexpr int MAX_CAND = 1024;
__global__ void __launch_bounds__(1024) sample_kernel(const SampleParams p) {
    __shared__ unsigned s_hist[256];
    __shared__ unsigned long long s_keys[MAX_CAND];
    __shared__ float s_scan[MAX_CAND];
    __shared__ unsigned s_prefix, s_need, s_count, s_eq_count;
    __shared__ float s_warp[32];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* lg = p.logits + (size_t)row * p.stride;
    const bool merging = p.merge_pairs != nullptr;
    const int n_items = merging ? p.merge_ranks * p.merge_k : p.vocab;
    // entry i of this row: its value and the token id it stands for
    auto pair_at = [&](int i) {
        const int w = i / p.merge_k, j = i - w * p.merge_k;
        return p.merge_pairs + (((size_t)w * p.rows + row) * p.merge_k + j) * 2;
    };
    auto val_at = [&](int i) { return merging ? __int_as_float(pair_at(i)[0]) : lg[i]; };
    auto id_at = [&](int i) { return merging ? (unsigned)pair_at(i)[1] : (unsigned)(i + p.idx_offset); };
    const float temp = p.temperature ? p.temperature[row] : 1.0f;
    int k = p.top_k ? p.top_k[row] : 0;
    const float top_p = p.top_p ? p.top_p[row] : 1.0f;
    const bool greedy = !p.cand_out && (temp <= 0.f || k == 1);
    if (k <= 0 || k > MAX_CAND) k = MAX_CAND;
    if (p.cand_out) k = p.cand_k;
    if (k > n_items) k = n_items;
    if (greedy) k = 1;
    // ---- radix select of the k-th largest key ----
    if (tid == 0) { s_prefix = 0; s_need = k; }
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) s_hist[tid] = 0;
        __syncthreads();
        const unsigned prefix = s_prefix;
        const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < n_items; i += 1024) {
            const unsigned key = order_key(val_at(i));
            if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 0xff], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            unsigned need = s_need, b = 255;
            for (;; --b) {
                const unsigned c = s_hist[b];
                if (c >= need || b == 0) break;
                need -= c;
            }
            s_prefix = prefix | (b << shift);
            s_need = need;
        }
        __syncthreads();
    }
    const unsigned thr = s_prefix;              // key of the k-th largest element
    const unsigned eq_quota = s_need;           // how many elements equal to thr are still needed
    if (tid == 0) { s_count = 0; s_eq_count = 0; }
    for (int i = tid; i < MAX_CAND; i += 1024) s_keys[i] = 0ull;
    __syncthreads();
    for (int i = tid; i < n_items; i += 1024) {
        const unsigned key = order_key(val_at(i));
        bool take = key > thr;
        if (key == thr) take = atomicAdd(&s_eq_count, 1u) < eq_quota;
        if (take) {
            const unsigned slot = atomicAdd(&s_count, 1u);
            if (slot < MAX_CAND) s_keys[slot] = ((unsigned long long)key << 32) | (0xffffffffu - id_at(i));
        }
    }
    __syncthreads();
    // ---- bitonic sort, descending (largest key first; ties -> lower token id first) ----
    for (int size = 2; size <= MAX_CAND; size <<= 1) {
        for (int strd = size >> 1; strd > 0; strd >>= 1) {
            const int i = tid, j = i ^ strd;
            if (j > i) {
                const unsigned long long a = s_keys[i], b = s_keys[j];
                const bool desc = (i & size) == 0;
                if ((a < b) == desc) { s_keys[i] = b; s_keys[j] = a; }
            }
            __syncthreads();
        }
    }
    const int n = min((int)s_count, k);
    if (p.cand_out) {
        // pass 1 of a sharded head: the best cand_k entries in order, padded with (-inf, no token)
        for (int i = tid; i < p.cand_k; i += 1024) {
            int* o = p.cand_out + ((size_t)row * p.cand_k + i) * 2;
            o[0] = i < n ? __float_as_int(key_to_float((unsigned)(s_keys[i] >> 32))) : (int)0xff800000u;
            o[1] = i < n ? (int)(0xffffffffu - (unsigned)(s_keys[i] & 0xffffffffu)) : 0x7fffffff;
        }
        return;
    }
    if (p.probs_out) {
        float* po = p.probs_out + (size_t)row * p.vocab;
        for (int i = tid; i < p.vocab; i += 1024) po[i] = 0.f;
    }
    __syncthreads();
    if (greedy) {
        if (tid == 0) {
            const int tok = (int)(0xffffffffu - (unsigned)(s_keys[0] & 0xffffffffu));
            p.tokens[row] = tok;
            if (p.probs_out) p.probs_out[(size_t)row * p.vocab + tok] = 1.0f;
        }
        return;
    }
    // ---- softmax over candidates (temperature applied here), inclusive scan ----
    const float vmax = key_to_float((unsigned)(s_keys[0] >> 32));
    float pr = 0.f;
    if (tid < n) pr = __expf((key_to_float((unsigned)(s_keys[tid] >> 32)) - vmax) / temp);
    float sc = pr;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, sc, o);
        if ((tid & 31) >= o) sc += t;
    }
    if ((tid & 31) == 31) s_warp[tid >> 5] = sc;
    __syncthreads();
    if (tid < 32) {
        float w = s_warp[tid];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, w, o);
            if (tid >= o) w += t;
        }
        s_warp[tid] = w;
    }
    __syncthreads();
    const float incl = sc + ((tid >> 5) > 0 ? s_warp[(tid >> 5) - 1] : 0.f);
    const float total = s_warp[31];
    // top-p: keep candidate i while the mass before it is < top_p * total (always keeps the first)
    const float before = incl - pr;
    const bool keep = tid < n && (top_p >= 1.0f || before < top_p * total || tid == 0);
    s_scan[tid] = keep ? incl : -1.0f;
    __syncthreads();
    // kept candidates form a prefix; its last inclusive value is the new normaliser
    __shared__ float s_z;
    __shared__ int s_nkeep;
    if (tid < n && keep && (tid == n - 1 || s_scan[tid + 1] < 0.f)) { s_z = incl; s_nkeep = tid + 1; }
    __syncthreads();
    const float z = s_z;
    const int nkeep = s_nkeep;
    if (p.probs_out && tid < nkeep) {
        const int tok = (int)(0xffffffffu - (unsigned)(s_keys[tid] & 0xffffffffu));
        p.probs_out[(size_t)row * p.vocab + tok] = pr / z;
    }
    const float u = uniform01(p.seeds ? p.seeds[row] : 0ull, (uint64_t)(p.step ? p.step[row] : 0)) * z;
    // first kept candidate whose inclusive mass reaches u
    __shared__ int s_pick;
    if (tid == 0) s_pick = nkeep - 1;
    __syncthreads();
    if (tid < nkeep && incl >= u && (tid == 0 || before < u)) atomicMin(&s_pick, tid);
    __syncthreads();
    if (tid == 0) p.tokens[row] = (int)(0xffffffffu - (unsigned)(s_keys[s_pick] & 0xffffffffu));
}
cudaError_t launch_sample(const SampleParams& p, cudaStream_t st) {
    if (p.rows == 0) return cudaSuccess;
    sample_kernel<<<p.rows, 1024, 0, st>>>(p);
    return cudaGetLastError();
}

// Presence / frequency penalties from a dense per-lane count table: counts[lane][t] = how often token t of this rank's
// vocabulary shard occurs in the lane's prompt + output so far (16-bit, saturating).  logits[row][t] -= presence[row] *
// (count > 0) + frequency[row] * count.  The table lives on the device and is advanced by count_tokens_kernel right after
// sampling, so a decode step with penalties needs nothing from the host and replays as a CUDA graph (reference:
// cuda_apply_logit_penalties_f32, src/v2/kernels/cuda/ops/CUDASamplingKernels.cu:5410, which takes the history per call).
__global__ void penalties_dense_kernel(float* logits, int stride, int vocab, const unsigned short* counts, int counts_stride,
                                       const float* presence, const float* frequency) {
    const int row = blockIdx.y;
    const float pp = presence[row], fp = frequency[row];
    if (pp == 0.f && fp == 0.f) return;
    const unsigned short* c = counts + (size_t)row * counts_stride;
    float* l = logits + (size_t)row * stride;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        const unsigned n = c[i];
        if (n) l[i] -= pp + fp * (float)n;
    }
}
cudaError_t launch_penalties_dense(float* logits, int rows, int vocab, int stride, const unsigned short* counts, int counts_stride,
                                   const float* presence, const float* frequency, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    penalties_dense_kernel<<<dim3(32, rows), 256, 0, st>>>(logits, stride, vocab, counts, counts_stride, presence, frequency);
    return cudaGetLastError();
}
// counts[row][tokens[row] - v0] += 1 for the tokens that fall into this shard (one thread per row; rows own their table rows)
__global__ void count_tokens_kernel(unsigned short* counts, int counts_stride, const int* tokens, int v0, int vocab, int rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int t = tokens[r] - v0;
    if (t < 0 || t >= vocab) return;
    unsigned short* c = counts + (size_t)r * counts_stride + t;
    if (*c < 32767) *c = *c + 1;
}
cudaError_t launch_count_tokens(unsigned short* counts, int counts_stride, const int* tokens, int v0, int vocab, int rows, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    count_tokens_kernel<<<(rows + 63) / 64, 64, 0, st>>>(counts, counts_stride, tokens, v0, vocab, rows);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// NaN / Inf scan
// ------------------------------------------------------------------------------------------------
__global__ void nan_scan_kernel(const void* x, size_t n, int dtype, int* counts) {
    int nn = 0, ni = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = dtype == 0 ? static_cast<const float*>(x)[i] : __bfloat162float(static_cast<const __nv_bfloat16*>(x)[i]);
        nn += isnan(v) ? 1 : 0;
        ni += isinf(v) ? 1 : 0;
    }
    nn = __reduce_add_sync(0xffffffffu, nn);
    ni = __reduce_add_sync(0xffffffffu, ni);
    if ((threadIdx.x & 31) == 0) {
        if (nn) atomicAdd(&counts[0], nn);
        if (ni) atomicAdd(&counts[1], ni);
    }
}
cudaError_t launch_nan_scan(const void* x, size_t n, int dtype, int* counts, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    const unsigned grid = (unsigned)min((size_t)1184, (n + 255) / 256);
    nan_scan_kernel<<<grid, 256, 0, st>>>(x, n, dtype, counts);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// speculative decoding verification
// ------------------------------------------------------------------------------------------------
__global__ void spec_verify_greedy_kernel(const int* draft, const int* target, int batch, int depth, int* n_accept, int* out_tokens) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    int n = 0;
    while (n < depth && draft[b * depth + n] == target[b * (depth + 1) + n]) ++n;
    n_accept[b] = n;
    for (int i = 0; i <= depth; ++i) out_tokens[b * (depth + 1) + i] = i <= n ? target[b * (depth + 1) + i] : -1;
}
cudaError_t launch_spec_verify_greedy(const int* draft, const int* target, int batch, int depth, int* n_accept,
                                      int* out_tokens, cudaStream_t st) {
    if (batch == 0) return cudaSuccess;
    spec_verify_greedy_kernel<<<(batch + 63) / 64, 64, 0, st>>>(draft, target, batch, depth, n_accept, out_tokens);
    return cudaGetLastError();
}

// block-wide inverse-CDF sample from w[i] = max(a[i] - b[i], 0) (b may be null); returns the index to all threads
LLM_DEVICE int block_sample_residual(const float* a, const float* b, int vocab, float u01, float* s_buf /*[blockDim.x + 1]*/) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int seg = (vocab + nt - 1) / nt;
    const int lo = min(tid * seg, vocab), hi = min(lo + seg, vocab);
    float s = 0.f;
    for (int i = lo; i < hi; ++i) s += fmaxf(a[i] - (b ? b[i] : 0.f), 0.f);
    s_buf[tid] = s;
    __syncthreads();
    if (tid == 0) {                    // serial scan over <= 1024 partials: negligible next to the vocab pass
        float run = 0.f;
        for (int t = 0; t < nt; ++t) { const float v = s_buf[t]; s_buf[t] = run; run += v; }
        s_buf[nt] = run;
    }
    __syncthreads();
    const float total = s_buf[nt];
    __shared__ int s_idx;
    if (tid == 0) s_idx = -1;
    __syncthreads();
    if (total > 0.f) {
        const float target = u01 * total;
        const float mine = s_buf[tid];
        const float next = (tid + 1 < nt) ? s_buf[tid + 1] : total;
        if (hi > lo && target >= mine && (target < next || tid == nt - 1 || next >= total)) {
            float run = mine;
            int pick = -1;
            for (int i = lo; i < hi; ++i) {
                const float w = fmaxf(a[i] - (b ? b[i] : 0.f), 0.f);
                run += w;
                if (w > 0.f) { pick = i; if (run > target) break; }
            }
            if (pick >= 0) atomicMax(&s_idx, pick);
        }
    }
    __syncthreads();
    int r = s_idx;
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(1024) spec_verify_reject_kernel(const SpecRejectParams p) {
    __shared__ float s_buf[1025];
    const int b = blockIdx.x;
    const uint64_t seed = p.seeds ? p.seeds[b] : 0ull;
    const uint64_t step = p.step ? (uint64_t)p.step[b] : 0ull;
    int n = 0;
    for (; n < p.depth; ++n) {
        const int x = p.draft[b * p.depth + n];
        const float pt = p.p_target[((size_t)b * (p.depth + 1) + n) * p.vocab + x];
        const float pd = p.p_draft[((size_t)b * p.depth + n) * p.vocab + x];
        const float r = uniform01(seed, step * 64 + 2 * n + 1);
        const bool accept = pd <= 0.f ? pt > 0.f : r * pd < pt;        // r < min(1, pt / pd)
        if (!accept) break;
        if (threadIdx.x == 0) p.out_tokens[b * (p.depth + 1) + n] = x;
    }
    const float* pt = p.p_target + ((size_t)b * (p.depth + 1) + n) * p.vocab;
    const float* pd = n < p.depth ? p.p_draft + ((size_t)b * p.depth + n) * p.vocab : nullptr;
    int tok = block_sample_residual(pt, pd, p.vocab, uniform01(seed, step * 64 + 2 * n + 2), s_buf);
    if (tok < 0) tok = block_sample_residual(pt, nullptr, p.vocab, uniform01(seed, step * 64 + 2 * n + 2), s_buf);
    if (threadIdx.x == 0) {
        p.out_tokens[b * (p.depth + 1) + n] = tok < 0 ? 0 : tok;
        for (int i = n + 1; i <= p.depth; ++i) p.out_tokens[b * (p.depth + 1) + i] = -1;
        p.n_accept[b] = n;
    }
}
cudaError_t launch_spec_verify_reject(const SpecRejectParams& p, cudaStream_t st) {
    if (p.batch == 0) return cudaSuccess;
    spec_verify_reject_kernel<<<p.batch, 1024, 0, st>>>(p);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// MoE router: softmax over all experts, top-k (ties -> lower id), optional renormalisation.
// One warp per token, up to 256 experts.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) moe_topk_kernel(const float* __restrict__ logits, int tokens, int n_experts, int k, int renorm,
                                                       int* __restrict__ ids, float* __restrict__ weights, int* __restrict__ counts) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= tokens) return;
    constexpr int PER = 8;
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * 32 + lane;
        v[j] = e < n_experts ? logits[(size_t)t * n_experts + e] : -INFINITY;
        mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) { v[j] = (j * 32 + lane) < n_experts ? __expf(v[j] - mx) : -1.0f; sum += fmaxf(v[j], 0.f); }
    sum = warp_sum(sum);
    float wsum = 0.f;
    float my_w = 0.f;
    int my_id = 0;
    for (int s = 0; s < k; ++s) {
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
        if ((bi & 31) == lane) v[bi >> 5] = -2.0f;          // remove the winner
        const float pw = best / sum;
        wsum += pw;
        if (lane == s) { my_w = pw; my_id = bi; }
    }
    if (lane < k) {
        ids[(size_t)t * k + lane] = my_id;
        weights[(size_t)t * k + lane] = renorm ? my_w / wsum : my_w;
        if (counts) atomicAdd(&counts[my_id], 1);
    }
}
cudaError_t launch_moe_topk(const float* logits, int tokens, int n_experts, int k, int renorm, int* ids, float* weights,
                            int* counts, cudaStream_t st) {
    if (tokens == 0) return cudaSuccess;
    if (n_experts > 256 || k > 32) return cudaErrorInvalidValue;
    moe_topk_kernel<<<(tokens + 3) / 4, 128, 0, st>>>(logits, tokens, n_experts, k, renorm, ids, weights, counts);
    return cudaGetLastError();
}

}  // namespace llm
