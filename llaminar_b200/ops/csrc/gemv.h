// Host-side declarations of the kernel launchers (implemented in the .cu files of this folder).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace llm {

struct TpFuse;   // tp_fuse.cuh

enum GemvEpilogue : int { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_MOE_COMBINE = 3 };

// One unit of grouped expert work: up to four (token, slot) pairs routed to the same local expert.
struct MoeItem {
    int expert;                // local expert index
    int m;                     // valid pairs (0: placeholder that only keeps the combine protocol alive)
    int slot[4];               // flat pair index = token * top_k + slot
};

// Weighted combine of the routed experts' outputs (EPI_MOE_COMBINE): the CTA that finishes a 128-column tile last sums
// weight * expert output over the locally owned pairs of every token, all-reduces the tile across the expert-parallel
// ranks (when `tp` is set) and adds the result to the residual stream.
struct MoeCombine {
    const int* ids;            // [tokens, top_k] global expert ids
    const float* wts;          // [tokens, top_k] routing weights
    int tokens, top_k, e0, n_local;
    float* yslot;              // [tokens * top_k, y_stride] per-pair expert outputs
    int y_stride;
    unsigned* tile_tickets;    // [n_tiles], zero between calls
    float* h;                  // fp32 residual stream [tokens, h_stride]
    int h_stride;
};

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
    const MoeItem* items;      // optional grouped-expert work list: blockIdx.z indexes it, rows come from the pairs
    const int* n_items;        // device count of valid items (CTAs beyond it exit)
    int x_div;                 // activation row of a pair = pair index / x_div
    MoeCombine moe;            // EPI_MOE_COMBINE only
    const TpFuse* tp;          // EPI_RESID only: device copy of the tensor-parallel descriptor -> the epilogue all-reduces
                               // the tile across ranks before adding it to the residual (nullptr: single rank)
};

cudaError_t launch_gemv(const GemvParams& p, int m_tile, int z, cudaStream_t st);
// Streaming kernel for plain dense calls (gemv_stream.cu): one persistent CTA per SM, chunks by bulk copy.  Returns
// cudaErrorNotSupported for calls it does not take (grouped experts, fused tensor-parallel epilogue, missing scratch).
cudaError_t launch_gemv_stream(const GemvParams& p, int m, float* partials, size_t partials_floats, unsigned* tickets, int* status, cudaStream_t st);
int gemv_pick_ksplit(int n_tiles, int k_blocks, int z);

struct MoeRouteParams {
    const float* h;            // fp32 residual stream [tokens, h_stride]
    int h_stride;
    const float* norm_w;       // RMSNorm gain applied before routing
    float eps;
    const __nv_bfloat16* router;   // [n_experts, d]
    int tokens, d, n_experts, top_k, renorm;
    int e0, n_local;           // expert range owned by this rank
    int* ids;                  // out [tokens, top_k]
    float* wts;                // out [tokens, top_k]
    MoeItem* items;            // out work list (capacity max_items)
    int* n_items;              // out
    int max_items;
    unsigned* ticket;          // one counter, zero between calls
    int* counts;               // optional out [n_local] pairs per local expert
    __nv_bfloat16* xn_out;     // optional out [tokens, d]: the normalised rows as bf16 (input of the grouped expert GEMMs)
};
cudaError_t launch_moe_combine_sorted(float* h, int h_stride, const float* y, const int* pos, const float* wts, int tokens, int top_k, int d,
                                      cudaStream_t st);
cudaError_t launch_moe_route(const MoeRouteParams& p, cudaStream_t st);

cudaError_t launch_dequant(int fmt, const uint8_t* w, int n, int k, __nv_bfloat16* out, cudaStream_t st);
cudaError_t launch_gather_rows(int fmt, const uint8_t* w, int k, const int* rows, int n_rows, float* out_f32,
                               __nv_bfloat16* out_bf16, int out_stride, cudaStream_t st);

}  // namespace llm
