// Tensor-core GEMM over quantised weight chunks (tcgen05 / TMEM / TMA): host-side interface.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace llm {

struct TpFuse;   // tp_fuse.cuh

struct GemmTcParams {
    const uint8_t* w;          // weight chunks [n_tiles][k_blocks][chunk]
    int fmt;
    int n, k, m;               // out[m, n] = sum_k x[m, k] * W[n, k]
    const __nv_bfloat16* x;    // [m, k] contiguous bf16
    void* out;                 // bf16 or fp32 [m, out_stride]; EPI_RESID: fp32 updated in place
    int out_stride;
    int out_f32;
    int epi;                   // GemvEpilogue values (store / residual add / SwiGLU)
    const float* bias;         // optional [n]
    float* accum;              // split-K scratch fp32 [m_pad][accum_stride], zero between calls
    unsigned* tickets;         // split-K counters [n_tiles * m_tiles], zero between calls
    int accum_stride;
    int ksplit;                // 0 = automatic
    int* status;               // optional device word: set to STATUS_TIMEOUT if a pipeline wait gave up
    int* debug;                // optional trace buffer (progress markers / ns timestamps written by the kernels); nullptr in production
    const TpFuse* tp;          // EPI_RESID in the small-batch kernel: fused cross-rank all-reduce of each tile (nullptr: off)
    int flags;                 // bit 1 (set by the launcher): stream-K work split in the small-batch kernel
};

cudaError_t launch_gemm_tc(const GemmTcParams& p, cudaStream_t st);
// small-batch kernel (block_m 32 or 64), implemented in gemm_tc_small.cu
cudaError_t launch_gemm_tc_small(const GemmTcParams& p, int block_m, int ksplit, cudaStream_t st);
// tokens per CTA tile and split factor the launcher would use (for sizing scratch)
void gemm_tc_plan(int m, int n, int k, int ksplit_hint, int* block_m, int* ksplit);

}  // namespace llm
