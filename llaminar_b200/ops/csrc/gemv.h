// Host-side declarations of the kernel launchers (implemented in the .cu files of this folder).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace llm {

struct TpFuse;   // tp_fuse.cuh

enum GemvEpilogue : int { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2 };

struct GemvParams {
    const uint8_t* w;          // weight chunks [n_tiles][k_blocks][chunk]
    int fmt;
    int n, k, n_tiles, k_blocks;
    const void* x;             // [rows, k]: fp32 when norm_w != nullptr, else bf16
    int x_stride;              // elements between activation rows
    int z_per_x;               // consecutive grid.z groups that share one activation row group (MoE slots)
    const float* norm_w;       // fused RMSNorm gain (nullptr: input is used as is)
    float eps;
    float* accum;              // split-K scratch: fp32 [rows][accum_stride], zero between calls
    unsigned* tickets;         // split-K arrival counters [z][n_tiles], zero between calls
    int accum_stride;
    int ksplit;                // 0 = choose automatically
    int epi;                   // GemvEpilogue
    void* out;                 // bf16 or fp32 [rows, out_stride]; EPI_RESID: fp32 residual updated in place
    int out_stride;
    int out_f32;
    const float* bias;         // optional [n]
    const int* expert_ids;     // optional [z]: weight matrix index per grid.z group
    size_t expert_stride;      // bytes between expert matrices
    const TpFuse* tp;          // EPI_RESID only: device copy of the tensor-parallel descriptor -> the epilogue all-reduces
                               // the tile across ranks before adding it to the residual (nullptr: single rank)
};

cudaError_t launch_gemv(const GemvParams& p, int m_tile, int z, cudaStream_t st);
int gemv_pick_ksplit(int n_tiles, int k_blocks, int z);
cudaError_t launch_dequant(int fmt, const uint8_t* w, int n, int k, __nv_bfloat16* out, cudaStream_t st);
cudaError_t launch_gather_rows(int fmt, const uint8_t* w, int k, const int* rows, int n_rows, float* out_f32,
                               __nv_bfloat16* out_bf16, int out_stride, cudaStream_t st);

}  // namespace llm
