// Launchers of the non-GEMM kernels (attention, norms, RoPE + KV append, sampling, debug scans).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace llm {

struct AttnDecodeParams {
    const __nv_bfloat16* q;        // [batch * rows_per_seq, n_heads, head_dim]
    const __nv_bfloat16* kv;       // [n_pages, 2, n_kv_heads, 64, head_dim]
    __nv_bfloat16* out;            // same shape as q
    const int* block_table;        // [batch, max_pages]
    const int* seq_lens;           // [batch] tokens in the cache including the rows of this step
    float* part_o;                 // split scratch [batch, n_kv_heads, splits, 16, head_dim]
    float* part_ml;                // split scratch [batch, n_kv_heads, splits, 16, 2]
    unsigned* tickets;             // [batch * n_kv_heads], zero between calls
    int n_heads, n_kv_heads, head_dim, max_pages, rows_per_seq;
    float scale;
    int n_pages;                   // pages of the cache (bounds-check build)
    // 8-bit cache (`kv` then points at bytes): a page is [2][n_kv_heads][64][head_dim] int8 followed by
    // [2][n_kv_heads][64][head_dim / 32] fp16 block scales (value = scale * int8)
    int kv_q8;
    size_t page_bytes, scale_off;
};

struct AttnPrefillParams {
    const __nv_bfloat16* q;        // [total_q, n_heads, head_dim]
    const __nv_bfloat16* kv;
    __nv_bfloat16* out;
    const int* block_table;        // [n_seqs, max_pages]
    const int* cu_q;               // [n_seqs + 1] prefix sums of query rows
    const int* ctx_lens;           // [n_seqs] tokens already cached before this chunk
    int n_heads, n_kv_heads, head_dim, max_pages;
    float scale;
    int n_pages;                   // pages of the cache (bounds-check build)
};

int attn_decode_pick_splits(int batch, int n_kv_heads, int max_pages_in_use);
cudaError_t launch_attn_decode(const AttnDecodeParams& p, int batch, int n_splits, cudaStream_t st);
cudaError_t launch_attn_prefill(const AttnPrefillParams& p, int n_seqs, int max_q_len, cudaStream_t st);
// tcgen05 version (head_dim 128 only); `status` (optional) receives STATUS_TIMEOUT if a pipeline wait gave up
cudaError_t launch_attn_prefill_tc(const AttnPrefillParams& p, int n_seqs, int max_q_len, int* status, cudaStream_t st);

struct RopeKVParams {
    __nv_bfloat16* qkv;            // [T, (n_heads + 2 n_kv_heads) * head_dim]; Q part is rewritten in place
    __nv_bfloat16* q_out;          // [T, n_heads, head_dim]
    __nv_bfloat16* kv;             // paged cache of this layer
    const float* q_norm;           // [head_dim] or nullptr
    const float* k_norm;
    const int* positions;          // [T]
    const int* seq_ids;            // [T] row of block_table for each token
    const int* block_table;        // [n_seqs, max_pages]
    int n_tokens, n_heads, n_kv_heads, head_dim, max_pages;
    float theta, eps;
    int n_pages, n_seqs;           // pages of the cache, rows of block_table (bounds-check build)
    int kv_q8;                     // 8-bit cache: rows are quantised per 32 values on the way in (layout: AttnDecodeParams)
    size_t page_bytes, scale_off;
};
// 8-bit cache -> bf16 pages for the prefill kernels: page j of sequence s (j < pages_of[s]) goes to staging page s * max_pages + j
cudaError_t launch_kv_dequant_pages(const uint8_t* kv8, size_t page_bytes, size_t scale_off, const int* block_table, const int* n_tokens,
                                    int n_seqs, int max_pages, int n_kv_heads, int head_dim, int n_pages, __nv_bfloat16* staging, cudaStream_t st);
// Gated-DeltaNet decode step (gdn.cu).  `in` is the row-major output of the block's input projection: columns [0, C) hold
// q | k | v, z_off / ab_off give the first column of the gate z and of the (alpha | b) pair; y = conv + SiLU of the q | k | v part.
struct GdnStepParams {
    const float* y;                 // [rows, C] fp32
    int C;
    const __nv_bfloat16* in;        // [rows, in_stride]
    int in_stride, z_off, ab_off;
    const float *ssm_a, *dt_bias, *norm_w;
    float* rec;                     // [slots, n_v, d, d]
    const int* slots;               // [rows]
    __nv_bfloat16* out;             // [rows, out_stride]
    int out_stride;
    int n_k, n_v, v_head_offset;
    float eps;
};
cudaError_t launch_gdn_conv_step(const __nv_bfloat16* in, int in_stride, const float* w, float* conv_state, const int* slots, float* y,
                                 int rows, int C, int K, cudaStream_t st);
cudaError_t launch_gdn_recurrent_step(const GdnStepParams& p, int rows, int d, cudaStream_t st);
// status word of the bounds-check build, per translation unit (0 in the production build)
int bounds_status_ops(bool reset);
int bounds_status_attention(bool reset);
int bounds_status_attention_tc(bool reset);
cudaError_t launch_rope_kv(const RopeKVParams& p, cudaStream_t st);

// h (+= delta) ; out = RMSNorm(h) * w   (fp32 residual stream, bf16 normalised output)
cudaError_t launch_rs_reduce_norm(const __nv_bfloat16* inbox, const unsigned* flags, unsigned target, int world, int rows_per_rank, int n_cap,
                                  int block_m, float* h, const float* norm_w, __nv_bfloat16* xn, int rows, int d, float eps,
                                  unsigned spin_limit, int* status, cudaStream_t st);
cudaError_t launch_rmsnorm(const float* h, const float* w, __nv_bfloat16* out, int rows, int d, float eps, cudaStream_t st);
cudaError_t launch_mtp_concat_norm(const float* emb, const float* hidden, const float* enorm, const float* hnorm,
                                   __nv_bfloat16* out, int rows, int d, float eps, cudaStream_t st);
// out[t, c] = silu(gate) * up, reading a gate|up GEMM output whose 32-column groups hold 16 gate + 16 up columns

// greedy: argmax of each row -> tokens[row]
cudaError_t launch_argmax(const float* logits, int rows, int vocab, int stride, int* tokens, int* pairs, int idx_offset,
                          cudaStream_t st);
cudaError_t launch_argmax_merge(const int* gathered, int ranks, int rows, int* tokens, cudaStream_t st);
struct SampleParams {
    const float* logits; int rows, vocab, stride;
    const float* temperature;      // [rows]
    const int* top_k;              // [rows] (0 = off)
    const float* top_p;            // [rows] (>= 1 = off)
    const uint64_t* seeds;         // [rows]
    const int* step;               // [rows] decode step counter mixed into the RNG
    int* tokens;                   // [rows]
    float* probs_out;              // optional [rows, vocab] final distribution (speculative sampling)
    // Vocabulary-sharded heads sample in two launches.  Pass 1 (cand_out set): every rank writes the cand_k best entries of
    // its shard as (float bits, global token id) pairs [rows, cand_k, 2] and draws nothing.  Pass 2 (merge_pairs set): the
    // all-gathered pairs [merge_ranks, rows, merge_k, 2] are the "vocabulary"; ties still go to the lower token id, so the
    // token is the one a single launch over the full row would have drawn.
    int* cand_out = nullptr; int cand_k = 0; int idx_offset = 0;
    const int* merge_pairs = nullptr; int merge_ranks = 0, merge_k = 0;
};
cudaError_t launch_sample(const SampleParams& p, cudaStream_t st);
cudaError_t launch_penalties_dense(float* logits, int rows, int vocab, int stride, const unsigned short* counts, int counts_stride,
                                   const float* presence, const float* frequency, cudaStream_t st);
cudaError_t launch_count_tokens(unsigned short* counts, int counts_stride, const int* tokens, int v0, int vocab, int rows, cudaStream_t st);
// counts[0] = #NaN, counts[1] = #Inf
cudaError_t launch_nan_scan(const void* x, size_t n, int dtype /*0 f32, 1 bf16*/, int* counts, cudaStream_t st);

// speculative decoding: greedy verify. draft [B, d], target_tokens [B, d+1] -> n_accept[B], out_tokens [B, d+1]
cudaError_t launch_spec_verify_greedy(const int* draft, const int* target, int batch, int depth, int* n_accept,
                                      int* out_tokens, cudaStream_t st);
struct SpecRejectParams {
    const float* p_target;         // [B, d+1, vocab] target distributions
    const float* p_draft;          // [B, d, vocab] draft distributions
    const int* draft;              // [B, d]
    const uint64_t* seeds; const int* step;
    int batch, depth, vocab;
    int* n_accept; int* out_tokens;   // [B], [B, d+1]
};
cudaError_t launch_spec_verify_reject(const SpecRejectParams& p, cudaStream_t st);

// MoE router: logits [T, E] fp32 -> top-k ids / renormalised weights
cudaError_t launch_moe_topk(const float* logits, int tokens, int n_experts, int k, int renorm, int* ids, float* weights,
                            int* counts, cudaStream_t st);

}  // namespace llm
