// Gated-DeltaNet linear attention, one new token per sequence (the decode step of the hybrid qwen35 blocks).
//
// Two launches per block and step.  The first applies the short causal convolution + SiLU to the projected q | k | v row of
// every sequence and shifts the sequence's convolution window.  The second runs the delta rule for every (sequence, value
// head): it L2-normalises that head's q and k, decays the head's d x d state, applies the rank-one correction, reads the
// output through q and finishes with the gated RMSNorm.  A CTA holds one head of one sequence; thread j owns column j of
// the state (d registers), so the state is read once and written once per token: 2 * 4 * d * d bytes per (sequence, head),
// which is what bounds the step (196 MB per block at 32 sequences x 48 heads x d = 128).
// State lives in per-sequence slots that the engine hands out (slot index per batch row); padded rows of a captured step
// point at a scratch slot.
// (reference: cuda_gdn_recurrent_step / cuda_short_conv1d_decode / cuda_gated_rmsnorm in
//  src/v2/kernels/cuda/gdn/CUDAGatedDeltaNetKernels.cu; value head j reads key head (j + first local head) mod n_k.)
#include "common.cuh"
#include "ops.h"

namespace llm {

__global__ void __launch_bounds__(256) gdn_conv_step_kernel(const __nv_bfloat16* in, int in_stride, const float* __restrict__ w,
                                                            float* conv_state, const int* slots, float* y, int C, int K) {
    const int b = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c >= C) return;
    float* st = conv_state + ((size_t)slots[b] * C + c) * (K - 1);
    const float x = __bfloat162float(in[(size_t)b * in_stride + c]);
    const float* wc = w + (size_t)c * K;
    float acc = wc[K - 1] * x;
    for (int j = 0; j < K - 1; ++j) {
        const float s = st[j];
        acc += wc[j] * s;
        if (j > 0) st[j - 1] = s;                      // shift the window by one
    }
    st[K - 2] = x;
    y[(size_t)b * C + c] = acc / (1.f + __expf(-acc));
}

template <int D>
LLM_DEVICE float block_sum(float v, float* s_red) {
    v = warp_sum(v);
    if (D <= 32) return v;
    const int warp = threadIdx.x >> 5;
    __syncthreads();                                    // s_red may still be read from the previous reduction
    if ((threadIdx.x & 31) == 0) s_red[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) t += s_red[i];
    return t;
}

template <int D>
__global__ void __launch_bounds__(D) gdn_recurrent_step_kernel(const GdnStepParams p) {
    __shared__ float s_q[D], s_k[D], s_red[4];
    const int h = blockIdx.x, b = blockIdx.y, j = threadIdx.x;
    const int kh = (h + p.v_head_offset) % p.n_k;
    const int kd = p.n_k * D;
    const float* yb = p.y + (size_t)b * p.C;
    float q = yb[kh * D + j], k = yb[kd + kh * D + j];
    const float v = yb[2 * kd + h * D + j];
    const float ssq = block_sum<D>(q * q, s_red), ssk = block_sum<D>(k * k, s_red);
    q *= rsqrtf(ssq + 1e-6f) * rsqrtf((float)D);
    k *= rsqrtf(ssk + 1e-6f);
    s_q[j] = q;
    s_k[j] = k;
    __syncthreads();
    const __nv_bfloat16* ab = p.in + (size_t)b * p.in_stride + p.ab_off;
    const float alpha = __bfloat162float(ab[h]) + p.dt_bias[h];
    const float sp = alpha > 20.f ? alpha : log1pf(__expf(alpha));
    const float a = __expf(p.ssm_a[h] * sp);
    const float beta = 1.f / (1.f + __expf(-__bfloat162float(ab[p.n_v + h])));
    float* S = p.rec + (((size_t)p.slots[b] * p.n_v + h) * D) * D;            // [i][j], row i contiguous over j
    float col[D];
    float kvm = 0.f;
#pragma unroll
    for (int i = 0; i < D; ++i) {
        col[i] = a * S[(size_t)i * D + j];
        kvm += col[i] * s_k[i];
    }
    const float u = beta * (v - kvm);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < D; ++i) {
        col[i] += s_k[i] * u;
        o += col[i] * s_q[i];
        S[(size_t)i * D + j] = col[i];
    }
    const float sso = block_sum<D>(o * o, s_red);
    const float z = __bfloat162float(p.in[(size_t)b * p.in_stride + p.z_off + h * D + j]);
    const float r = o * rsqrtf(sso / D + p.eps) * p.norm_w[j] * (z / (1.f + __expf(-z)));
    p.out[(size_t)b * p.out_stride + h * D + j] = __float2bfloat16(r);
}

cudaError_t launch_gdn_conv_step(const __nv_bfloat16* in, int in_stride, const float* w, float* conv_state, const int* slots, float* y,
                                 int rows, int C, int K, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    if (K < 2 || K > 16) return cudaErrorInvalidValue;
    gdn_conv_step_kernel<<<dim3((C + 255) / 256, rows), 256, 0, st>>>(in, in_stride, w, conv_state, slots, y, C, K);
    return cudaGetLastError();
}

cudaError_t launch_gdn_recurrent_step(const GdnStepParams& p, int rows, int d, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    const dim3 grid(p.n_v, rows);
    switch (d) {
        case 32: gdn_recurrent_step_kernel<32><<<grid, 32, 0, st>>>(p); break;
        case 64: gdn_recurrent_step_kernel<64><<<grid, 64, 0, st>>>(p); break;
        case 128: gdn_recurrent_step_kernel<128><<<grid, 128, 0, st>>>(p); break;
        default: return cudaErrorNotSupported;
    }
    return cudaGetLastError();
}

}  // namespace llm
