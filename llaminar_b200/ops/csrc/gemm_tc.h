// Tensor-core GEMM over quantised weight chunks (tcgen05 / TMEM / TMA): host-side interface.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace llm {

struct TpFuse;   // tp_fuse.cuh

// All-gather fused into the activation path of the large-tile kernel (column-parallel QKV / gate|up on row-sharded
// input).  Rank r owns rows [r * rows_per_rank, (r + 1) * rows_per_rank) of x and keeps them in a symmetric-memory
// buffer.  A few copier CTAs at the head of the same launch pull all rows from their owners (peers over NVLink) with
// plain 16-byte loads into a local staging buffer, m-tile by m-tile in the order the other CTAs will need them (own
// rows first), while those CTAs already multiply the tiles that have landed; the tensor map reads only the local
// buffer, so no TMA touches peer memory.
struct AgFuse {
    const __nv_bfloat16* src[8];   // every rank's own-row buffer of this call's parity (symmetric memory; src[rank] is local)
    unsigned* avail[8];            // per rank: [8] counters; avail[r][s] = calls whose rows rank s has published to rank r
    __nv_bfloat16* stage;          // local [m, k] staging buffer that the tensor map reads
    unsigned* staged;              // local [m_tiles] counters of finished copy slices (zeroed by the launcher)
    int world, rank, rows_per_rank;
    int copy_ctas;                 // copier CTAs at the head of the grid
    unsigned epoch;                // earlier calls on this arena (identical on all ranks)
    unsigned spin_limit;
};

// Reduce-scatter fused into the epilogue of the large-tile kernel (row-parallel attention-output / FFN-down projections
// of a prefill chunk).  The residual stream is sharded by rows between the ranks: rank o owns rows [o * rows_per_rank,
// (o + 1) * rows_per_rank).  Every CTA converts its finished partial tile to bf16, transposes it through shared memory
// and writes it with 16-byte stores straight into the inbox of the rank that owns those rows (peer memory over NVLink, or
// local memory for its own rows), then bumps that rank's arrival counter for the tile's row block.  The transfers of a
// tile overlap the main loops of the CTAs that are still computing.  The owner sums the `world` partials of its rows,
// adds the residual and applies the next RMSNorm in `rs_reduce_norm` (ops.h), which waits (bounded) on the counters.
// No TMA touches peer memory and nothing is multicast.  The reference runs GEMM, ncclAllReduce and the add as three
// stages (reference: src/v2/models/qwen/QwenGraphBase.cpp:2937-3014).
struct RsFuse {
    __nv_bfloat16* inbox[8];   // per owner: [2 parities][world sources][rows_per_rank][n_cap] bf16 (symmetric memory)
    unsigned* flags[8];        // per owner: [2 parities][rows_per_rank / block_m] arrival counters (symmetric memory)
    int world, rank, rows_per_rank, n_cap;
    int parity;                // which half of inbox / flags this call uses (call counter & 1, identical on all ranks)
    int flags_per_parity;
};

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
    float* partials;           // small-batch kernel: [grid][2][32 tokens][128 rows] fp32 slots for split tiles (nullptr: atomics into accum)
    int ksplit;                // 0 = automatic
    int* status;               // optional device word: set to STATUS_TIMEOUT if a pipeline wait gave up
    int* debug;                // optional trace buffer (progress markers / ns timestamps written by the kernels); nullptr in production
    const TpFuse* tp;          // EPI_RESID in the small-batch kernel: fused cross-rank all-reduce of each tile (nullptr: off)
    int flags;                 // bit 1 (set by the launcher): stream-K work split in the small-batch kernel; with `debug`: 0x100 makes the
                               // large-tile kernel write per-CTA ns timestamps (8 x u64 per CTA) instead of progress markers, bits 8.. select
                               // the traced CTA of the small-batch kernel
    int ag_on;                 // large-tile kernel: x rows are gathered from the ranks of `ag` inside the launch
    AgFuse ag;
    int rs_on;                 // large-tile kernel: partial tiles go to the owners of their rows (`rs`) instead of `out`
    RsFuse rs;
    // Grouped mode of the large-tile kernel (expert GEMMs of a mixture-of-experts prefill chunk): `groups` weight matrices of the
    // same shape, `w_group_stride` bytes apart; the rows of x / out that belong to group g are [group_row_off[g],
    // group_row_off[g + 1]) (rows sorted by expert on the device).  blockIdx.y runs over the m-tiles of all groups,
    // group_tile_off[g] = tiles of the groups before g; the grid is sized from a host-side upper bound and surplus CTAs exit.
    int groups;
    const int* group_row_off;  // device [groups + 1]
    const int* group_tile_off; // device [groups + 1]
    long long w_group_stride;
    int group_bm;              // tile height the offsets were computed for
};

cudaError_t launch_gemm_tc(const GemmTcParams& p, cudaStream_t st);
// small-batch kernel (block_m 32 or 64), implemented in gemm_tc_small.cu
cudaError_t launch_gemm_tc_small(const GemmTcParams& p, int block_m, int ksplit, cudaStream_t st);
// tile height the launcher uses for a fused reduce-scatter launch of m rows (the owners' counters are per tile of that height)
int gemm_tc_rs_block_m(int m, int rows_per_rank);
// tokens per CTA tile and split factor the launcher would use (for sizing scratch)
void gemm_tc_plan(int m, int n, int k, int ksplit_hint, int* block_m, int* ksplit);

}  // namespace llm
