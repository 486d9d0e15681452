// pybind11 surface of the CUDA extension: thin argument checking + launch on the current torch stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "gemm_tc.h"
#include "gemv.h"
#include "ops.h"
#include "launch.h"

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

#define LLM_CUDA_CHECK(expr)                                                                         \
    do {                                                                                             \
        cudaError_t e__ = (expr);                                                                    \
        TORCH_CHECK(e__ == cudaSuccess, #expr " failed: ", cudaGetErrorString(e__));                 \
    } while (0)

static cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
template <class T> static const T* cptr(const OptTensor& t) { return t.has_value() ? static_cast<const T*>(t->data_ptr()) : nullptr; }
template <class T> static T* mptr(const OptTensor& t) { return t.has_value() ? static_cast<T*>(t->data_ptr()) : nullptr; }
static void check_cuda(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous() || t.stride(-1) == 1, name, " must have unit inner stride");
}

static void gemv(const Tensor& w, int64_t fmt, int64_t n, int64_t k, const Tensor& x, const OptTensor& norm_w, double eps,
                 Tensor out, int64_t epi, const OptTensor& bias, const OptTensor& accum, const OptTensor& tickets,
                 int64_t ksplit, const OptTensor& expert_ids, int64_t expert_stride, int64_t z_per_x, int64_t m_tile, int64_t z,
                 const OptTensor& tp, const OptTensor& partials, const OptTensor& status, bool stream) {
    check_cuda(w, "w"); check_cuda(x, "x"); check_cuda(out, "out");
    const c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(k % 256 == 0, "k must be a multiple of 256");
    llm::GemvParams p{};
    p.w = static_cast<const uint8_t*>(w.data_ptr());
    p.fmt = (int)fmt; p.n = (int)n; p.k = (int)k; p.n_tiles = (int)((n + 127) / 128); p.k_blocks = (int)(k / 256);
    p.x = x.data_ptr(); p.x_stride = (int)x.stride(0); p.z_per_x = (int)std::max<int64_t>(z_per_x, 1);
    if (norm_w.has_value()) {
        TORCH_CHECK(x.scalar_type() == torch::kFloat32, "fused-norm GEMV takes the fp32 residual stream");
        TORCH_CHECK(norm_w->scalar_type() == torch::kFloat32, "norm gain must be fp32");
    } else {
        TORCH_CHECK(x.scalar_type() == torch::kBFloat16, "GEMV input must be bf16");
    }
    p.norm_w = cptr<float>(norm_w); p.eps = (float)eps;
    p.accum = mptr<float>(accum); p.tickets = mptr<unsigned>(tickets);
    p.accum_stride = accum.has_value() ? (int)accum->stride(0) : 0;
    if (accum.has_value()) {
        TORCH_CHECK(accum->size(0) >= m_tile * z && accum->stride(0) >= p.n_tiles * 128, "split-K scratch too small");
        TORCH_CHECK(tickets.has_value() && tickets->numel() >= z * p.n_tiles, "ticket scratch too small");
    }
    p.ksplit = (int)ksplit; p.epi = (int)epi;
    p.out = out.data_ptr(); p.out_stride = (int)out.stride(0);
    p.out_f32 = out.scalar_type() == torch::kFloat32;
    if (epi == llm::EPI_RESID) TORCH_CHECK(p.out_f32, "residual epilogue updates an fp32 stream");
    if (epi == llm::EPI_SWIGLU) TORCH_CHECK(!p.out_f32, "SwiGLU epilogue writes bf16");
    p.bias = cptr<float>(bias);
    p.expert_ids = cptr<int>(expert_ids); p.expert_stride = (size_t)expert_stride;
    p.tp = tp.has_value() ? reinterpret_cast<const llm::TpFuse*>(tp->data_ptr()) : nullptr;
    if (stream && z == 1 && partials.has_value() && partials->scalar_type() == torch::kFloat32 && tickets.has_value() &&
        tickets->numel() >= p.n_tiles) {
        const cudaError_t e = llm::launch_gemv_stream(p, (int)m_tile, mptr<float>(partials), (size_t)partials->numel(), mptr<unsigned>(tickets),
                                                      status.has_value() ? static_cast<int*>(status->data_ptr()) : nullptr, cur_stream());
        if (e != cudaErrorNotSupported) { LLM_CUDA_CHECK(e); return; }
    }
    LLM_CUDA_CHECK(llm::launch_gemv(p, (int)m_tile, (int)z, cur_stream()));
}

// Router: RMSNorm + projection + softmax top-k + grouped work list of the local experts (moe_ep.cu).
static void moe_route(const Tensor& h, const Tensor& norm_w, double eps, const Tensor& router, int64_t top_k, bool renorm,
                      int64_t e0, int64_t n_local, Tensor ids, Tensor wts, Tensor items, Tensor n_items, Tensor ticket,
                      const OptTensor& counts) {
    check_cuda(h, "h"); check_cuda(router, "router");
    const c10::cuda::CUDAGuard guard(h.device());
    TORCH_CHECK(h.scalar_type() == torch::kFloat32 && router.scalar_type() == torch::kBFloat16 && router.is_contiguous());
    TORCH_CHECK(ids.scalar_type() == torch::kInt32 && wts.scalar_type() == torch::kFloat32 && items.scalar_type() == torch::kInt32);
    llm::MoeRouteParams p{};
    p.h = static_cast<const float*>(h.data_ptr()); p.h_stride = (int)h.stride(0);
    p.norm_w = static_cast<const float*>(norm_w.data_ptr()); p.eps = (float)eps;
    p.router = static_cast<const __nv_bfloat16*>(router.data_ptr());
    p.tokens = (int)h.size(0); p.d = (int)router.size(1); p.n_experts = (int)router.size(0);
    p.top_k = (int)top_k; p.renorm = renorm ? 1 : 0; p.e0 = (int)e0; p.n_local = (int)n_local;
    TORCH_CHECK(ids.numel() >= p.tokens * p.top_k && wts.numel() >= p.tokens * p.top_k);
    p.ids = static_cast<int*>(ids.data_ptr()); p.wts = static_cast<float*>(wts.data_ptr());
    p.items = reinterpret_cast<llm::MoeItem*>(items.data_ptr());
    p.max_items = (int)(items.numel() * 4 / sizeof(llm::MoeItem));
    p.n_items = static_cast<int*>(n_items.data_ptr()); p.ticket = static_cast<unsigned*>(ticket.data_ptr());
    p.counts = mptr<int>(counts);
    LLM_CUDA_CHECK(llm::launch_moe_route(p, cur_stream()));
}

// Routing only (any number of tokens): RMSNorm + router + softmax top-k; optionally the normalised rows as bf16.
static void moe_route_only(const Tensor& h, const Tensor& norm_w, double eps, const Tensor& router, int64_t top_k, bool renorm,
                           Tensor ids, Tensor wts, const OptTensor& xn_out) {
    check_cuda(h, "h"); check_cuda(router, "router");
    const c10::cuda::CUDAGuard guard(h.device());
    TORCH_CHECK(h.scalar_type() == torch::kFloat32 && router.scalar_type() == torch::kBFloat16 && router.is_contiguous());
    TORCH_CHECK(ids.scalar_type() == torch::kInt32 && wts.scalar_type() == torch::kFloat32);
    llm::MoeRouteParams p{};
    p.h = static_cast<const float*>(h.data_ptr()); p.h_stride = (int)h.stride(0);
    p.norm_w = static_cast<const float*>(norm_w.data_ptr()); p.eps = (float)eps;
    p.router = static_cast<const __nv_bfloat16*>(router.data_ptr());
    p.tokens = (int)h.size(0); p.d = (int)router.size(1); p.n_experts = (int)router.size(0);
    p.top_k = (int)top_k; p.renorm = renorm ? 1 : 0;
    TORCH_CHECK(ids.numel() >= (int64_t)p.tokens * p.top_k && wts.numel() >= (int64_t)p.tokens * p.top_k);
    p.ids = static_cast<int*>(ids.data_ptr()); p.wts = static_cast<float*>(wts.data_ptr());
    if (xn_out.has_value()) {
        TORCH_CHECK(xn_out->scalar_type() == torch::kBFloat16 && xn_out->is_contiguous() && xn_out->size(0) >= p.tokens && xn_out->size(1) == p.d);
        p.xn_out = static_cast<__nv_bfloat16*>(xn_out->data_ptr());
    }
    LLM_CUDA_CHECK(llm::launch_moe_route(p, cur_stream()));
}

static void moe_combine_sorted(Tensor h, const Tensor& y, const Tensor& pos, const Tensor& wts, int64_t top_k) {
    check_cuda(h, "h"); check_cuda(y, "y");
    const c10::cuda::CUDAGuard guard(h.device());
    TORCH_CHECK(h.scalar_type() == torch::kFloat32 && y.scalar_type() == torch::kFloat32 && y.is_contiguous() && h.stride(1) == 1);
    TORCH_CHECK(pos.scalar_type() == torch::kInt32 && wts.scalar_type() == torch::kFloat32 && pos.is_contiguous() && wts.is_contiguous());
    TORCH_CHECK(pos.numel() >= h.size(0) * top_k && wts.numel() >= h.size(0) * top_k && y.size(1) == h.size(1));
    LLM_CUDA_CHECK(llm::launch_moe_combine_sorted(static_cast<float*>(h.data_ptr()), (int)h.stride(0), static_cast<const float*>(y.data_ptr()),
                                                  static_cast<const int*>(pos.data_ptr()), static_cast<const float*>(wts.data_ptr()),
                                                  (int)h.size(0), (int)top_k, (int)h.size(1), cur_stream()));
}

// Grouped expert GEMM on the tensor cores: rows of x / out sorted by expert (see GemmTcParams::groups in gemm_tc.h).
static void gemm_tc_grouped(const Tensor& w, int64_t fmt, int64_t n, int64_t k, int64_t groups, int64_t w_group_stride, const Tensor& x, Tensor out,
                            int64_t epi, const Tensor& row_off, const Tensor& tile_off, int64_t bm, const OptTensor& status) {
    check_cuda(w, "w"); check_cuda(x, "x"); check_cuda(out, "out");
    const c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && x.is_contiguous(), "grouped GEMM input must be contiguous bf16");
    TORCH_CHECK(row_off.scalar_type() == torch::kInt32 && tile_off.scalar_type() == torch::kInt32 && row_off.is_cuda() && tile_off.is_cuda());
    TORCH_CHECK(row_off.numel() >= groups + 1 && tile_off.numel() >= groups + 1 && groups >= 1);
    TORCH_CHECK(epi == llm::EPI_STORE || epi == llm::EPI_SWIGLU, "grouped GEMM: store or SwiGLU epilogue");
    llm::GemmTcParams p{};
    p.w = static_cast<const uint8_t*>(w.data_ptr()); p.fmt = (int)fmt; p.n = (int)n; p.k = (int)k; p.m = (int)x.size(0);
    p.x = static_cast<const __nv_bfloat16*>(x.data_ptr());
    p.out = out.data_ptr(); p.out_stride = (int)out.stride(0); p.out_f32 = out.scalar_type() == torch::kFloat32;
    TORCH_CHECK(out.size(0) >= x.size(0), "grouped GEMM: out has fewer rows than x");
    p.epi = (int)epi; p.status = mptr<int>(status); p.ksplit = 1;
    p.groups = (int)groups; p.w_group_stride = (long long)w_group_stride; p.group_bm = (int)bm;
    p.group_row_off = static_cast<const int*>(row_off.data_ptr()); p.group_tile_off = static_cast<const int*>(tile_off.data_ptr());
    LLM_CUDA_CHECK(llm::launch_gemm_tc(p, cur_stream()));
}

// Grouped expert GEMV over the router's work list: epi = EPI_SWIGLU (gate|up) or EPI_MOE_COMBINE (down + combine [+ all-reduce]).
static void moe_gemv(const Tensor& w, int64_t fmt, int64_t n, int64_t k, int64_t expert_stride, const Tensor& x, const OptTensor& norm_w,
                     double eps, Tensor out, int64_t epi, const Tensor& items, const Tensor& n_items, int64_t x_div, int64_t z_max,
                     const OptTensor& accum, const OptTensor& tickets, const OptTensor& ids, const OptTensor& wts, int64_t top_k,
                     int64_t e0, int64_t n_local, const OptTensor& h, const OptTensor& tile_tickets, const OptTensor& tp) {
    check_cuda(w, "w"); check_cuda(x, "x"); check_cuda(out, "out");
    const c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(k % 256 == 0, "k must be a multiple of 256");
    llm::GemvParams p{};
    p.w = static_cast<const uint8_t*>(w.data_ptr());
    p.fmt = (int)fmt; p.n = (int)n; p.k = (int)k; p.n_tiles = (int)((n + 127) / 128); p.k_blocks = (int)(k / 256);
    p.x = x.data_ptr(); p.x_stride = (int)x.stride(0); p.z_per_x = 1;
    if (norm_w.has_value()) {
        TORCH_CHECK(x.scalar_type() == torch::kFloat32, "fused-norm GEMV takes the fp32 residual stream");
    } else {
        TORCH_CHECK(x.scalar_type() == torch::kBFloat16, "GEMV input must be bf16");
    }
    p.norm_w = cptr<float>(norm_w); p.eps = (float)eps;
    p.accum = mptr<float>(accum); p.tickets = mptr<unsigned>(tickets);
    p.accum_stride = accum.has_value() ? (int)accum->stride(0) : 0;
    if (accum.has_value()) {
        TORCH_CHECK(accum->size(0) >= 4 * z_max && accum->stride(0) >= p.n_tiles * 128, "split-K scratch too small");
        TORCH_CHECK(tickets.has_value() && tickets->numel() >= z_max * p.n_tiles, "ticket scratch too small");
    }
    p.epi = (int)epi;
    p.out = out.data_ptr(); p.out_stride = (int)out.stride(0); p.out_f32 = out.scalar_type() == torch::kFloat32;
    p.expert_stride = (size_t)expert_stride;
    p.items = reinterpret_cast<const llm::MoeItem*>(items.data_ptr());
    p.n_items = static_cast<const int*>(n_items.data_ptr());
    p.x_div = (int)x_div;
    TORCH_CHECK(z_max * (int64_t)sizeof(llm::MoeItem) <= items.numel() * 4, "work list shorter than the grid");
    if (epi == llm::EPI_MOE_COMBINE) {
        TORCH_CHECK(ids.has_value() && wts.has_value() && h.has_value() && tile_tickets.has_value(), "combine needs ids, weights, h, tickets");
        TORCH_CHECK(p.out_f32 && h->scalar_type() == torch::kFloat32);
        p.moe.ids = cptr<int>(ids); p.moe.wts = cptr<float>(wts);
        p.moe.tokens = (int)h->size(0); p.moe.top_k = (int)top_k; p.moe.e0 = (int)e0; p.moe.n_local = (int)n_local;
        p.moe.yslot = static_cast<float*>(out.data_ptr()); p.moe.y_stride = (int)out.stride(0);
        p.moe.tile_tickets = mptr<unsigned>(tile_tickets);
        TORCH_CHECK(tile_tickets->numel() >= p.n_tiles);
        p.moe.h = static_cast<float*>(h->data_ptr()); p.moe.h_stride = (int)h->stride(0);
        p.tp = tp.has_value() ? reinterpret_cast<const llm::TpFuse*>(tp->data_ptr()) : nullptr;
    } else {
        TORCH_CHECK(epi == llm::EPI_SWIGLU && !p.out_f32, "grouped gate|up writes bf16 through the SwiGLU epilogue");
    }
    LLM_CUDA_CHECK(llm::launch_gemv(p, 4, (int)z_max, cur_stream()));
}

static void dequant(const Tensor& w, int64_t fmt, int64_t n, int64_t k, Tensor out) {
    check_cuda(w, "w"); check_cuda(out, "out");
    const c10::cuda::CUDAGuard guard(w.device());
    TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.numel() >= n * k);
    LLM_CUDA_CHECK(llm::launch_dequant((int)fmt, static_cast<const uint8_t*>(w.data_ptr()), (int)n, (int)k,
                                       static_cast<__nv_bfloat16*>(out.data_ptr()), cur_stream()));
}

static void gather_rows(const Tensor& w, int64_t fmt, int64_t k, const Tensor& rows, Tensor out) {
    check_cuda(w, "w"); check_cuda(out, "out");
    const c10::cuda::CUDAGuard guard(w.device());
    TORCH_CHECK(rows.scalar_type() == torch::kInt32);
    const bool f32 = out.scalar_type() == torch::kFloat32;
    LLM_CUDA_CHECK(llm::launch_gather_rows((int)fmt, static_cast<const uint8_t*>(w.data_ptr()), (int)k,
                                           static_cast<const int*>(rows.data_ptr()), (int)rows.numel(),
                                           f32 ? static_cast<float*>(out.data_ptr()) : nullptr,
                                           f32 ? nullptr : static_cast<__nv_bfloat16*>(out.data_ptr()), (int)out.stride(0), cur_stream()));
}

static void rmsnorm(const Tensor& h, const Tensor& w, Tensor out, double eps) {
    check_cuda(h, "h");
    const c10::cuda::CUDAGuard guard(h.device());
    TORCH_CHECK(h.scalar_type() == torch::kFloat32 && out.scalar_type() == torch::kBFloat16 && h.is_contiguous() && out.is_contiguous());
    LLM_CUDA_CHECK(llm::launch_rmsnorm(static_cast<const float*>(h.data_ptr()), static_cast<const float*>(w.data_ptr()),
                                       static_cast<__nv_bfloat16*>(out.data_ptr()), (int)h.size(0), (int)h.size(1), (float)eps, cur_stream()));
}

static void mtp_concat_norm(const Tensor& emb, const Tensor& hidden, const Tensor& enorm, const Tensor& hnorm, Tensor out, double eps) {
    check_cuda(emb, "emb"); check_cuda(hidden, "hidden");
    const c10::cuda::CUDAGuard guard(emb.device());
    TORCH_CHECK(emb.scalar_type() == torch::kFloat32 && hidden.scalar_type() == torch::kFloat32 && out.scalar_type() == torch::kBFloat16);
    TORCH_CHECK(emb.is_contiguous() && hidden.is_contiguous() && out.is_contiguous() && emb.sizes() == hidden.sizes());
    TORCH_CHECK(out.size(0) == emb.size(0) && out.size(1) == 2 * emb.size(1));
    LLM_CUDA_CHECK(llm::launch_mtp_concat_norm(static_cast<const float*>(emb.data_ptr()), static_cast<const float*>(hidden.data_ptr()),
                                               static_cast<const float*>(enorm.data_ptr()), static_cast<const float*>(hnorm.data_ptr()),
                                               static_cast<__nv_bfloat16*>(out.data_ptr()), (int)emb.size(0), (int)emb.size(1), (float)eps,
                                               cur_stream()));
}

static void rope_kv(Tensor qkv, Tensor q_out, Tensor kv, const OptTensor& q_norm, const OptTensor& k_norm, const Tensor& positions,
                    const Tensor& seq_ids, const Tensor& block_table, int64_t n_heads, int64_t n_kv_heads, int64_t head_dim,
                    double theta, double eps) {
    check_cuda(qkv, "qkv");
    const c10::cuda::CUDAGuard guard(qkv.device());
    TORCH_CHECK(qkv.is_contiguous() && q_out.is_contiguous() && kv.is_contiguous());
    TORCH_CHECK(positions.scalar_type() == torch::kInt32 && seq_ids.scalar_type() == torch::kInt32 && block_table.scalar_type() == torch::kInt32);
    llm::RopeKVParams p{};
    p.qkv = static_cast<__nv_bfloat16*>(qkv.data_ptr()); p.q_out = static_cast<__nv_bfloat16*>(q_out.data_ptr());
    p.kv = static_cast<__nv_bfloat16*>(kv.data_ptr());
    if (kv.scalar_type() == torch::kUInt8) {           // 8-bit cache: [n_pages, page_bytes]
        TORCH_CHECK(kv.dim() == 2, "an 8-bit KV layer is [n_pages, page_bytes]");
        p.kv_q8 = 1; p.page_bytes = (size_t)kv.size(1); p.scale_off = (size_t)2 * n_kv_heads * 64 * head_dim;
        TORCH_CHECK(p.page_bytes == p.scale_off + p.scale_off / 16, "8-bit KV page size does not match heads x head_dim");
    } else {
        TORCH_CHECK(kv.scalar_type() == torch::kBFloat16, "KV cache must be bf16 or 8-bit");
    }
    p.q_norm = cptr<float>(q_norm); p.k_norm = cptr<float>(k_norm);
    p.positions = static_cast<const int*>(positions.data_ptr()); p.seq_ids = static_cast<const int*>(seq_ids.data_ptr());
    p.block_table = static_cast<const int*>(block_table.data_ptr());
    p.n_tokens = (int)qkv.size(0); p.n_heads = (int)n_heads; p.n_kv_heads = (int)n_kv_heads; p.head_dim = (int)head_dim;
    p.max_pages = (int)block_table.size(1); p.theta = (float)theta; p.eps = (float)eps;
    p.n_pages = (int)kv.size(0); p.n_seqs = (int)block_table.size(0);
    LLM_CUDA_CHECK(llm::launch_rope_kv(p, cur_stream()));
}

// 8-bit KV pages of the sequences in `block_table` -> bf16 staging pages (page j of sequence s at staging[s * max_pages + j])
static void kv_dequant_pages(const Tensor& kv8, const Tensor& block_table, const Tensor& n_tokens, int64_t n_kv_heads, int64_t head_dim,
                             Tensor staging) {
    check_cuda(kv8, "kv8"); check_cuda(staging, "staging");
    const c10::cuda::CUDAGuard guard(kv8.device());
    TORCH_CHECK(kv8.scalar_type() == torch::kUInt8 && kv8.dim() == 2 && kv8.is_contiguous());
    TORCH_CHECK(block_table.scalar_type() == torch::kInt32 && block_table.dim() == 2 && block_table.is_contiguous());
    TORCH_CHECK(n_tokens.scalar_type() == torch::kInt32 && n_tokens.numel() == block_table.size(0));
    TORCH_CHECK(staging.scalar_type() == torch::kBFloat16 && staging.is_contiguous());
    const size_t scale_off = (size_t)2 * n_kv_heads * 64 * head_dim;
    TORCH_CHECK((size_t)kv8.size(1) == scale_off + scale_off / 16, "8-bit KV page size does not match heads x head_dim");
    TORCH_CHECK(staging.numel() >= block_table.numel() * (int64_t)scale_off, "staging pool too small");
    LLM_CUDA_CHECK(llm::launch_kv_dequant_pages(static_cast<const uint8_t*>(kv8.data_ptr()), (size_t)kv8.size(1), scale_off,
                                                static_cast<const int*>(block_table.data_ptr()), static_cast<const int*>(n_tokens.data_ptr()),
                                                (int)block_table.size(0), (int)block_table.size(1), (int)n_kv_heads, (int)head_dim, (int)kv8.size(0),
                                                static_cast<__nv_bfloat16*>(staging.data_ptr()), cur_stream()));
}

// Linear-attention decode step, first launch: y = SiLU(conv(window | in[:, :C])), windows shifted (gdn.cu)
static void gdn_conv_step(const Tensor& in, const Tensor& conv_w, Tensor conv_state, const Tensor& slots, Tensor y) {
    check_cuda(in, "in"); check_cuda(conv_state, "conv_state");
    const c10::cuda::CUDAGuard guard(in.device());
    const int rows = (int)in.size(0), C = (int)conv_w.size(0), K = (int)conv_w.size(1);
    TORCH_CHECK(in.scalar_type() == torch::kBFloat16 && in.dim() == 2 && in.stride(1) == 1 && in.size(1) >= C);
    TORCH_CHECK(conv_w.scalar_type() == torch::kFloat32 && conv_w.is_contiguous());
    TORCH_CHECK(conv_state.scalar_type() == torch::kFloat32 && conv_state.is_contiguous() && conv_state.dim() == 3 &&
                conv_state.size(1) == C && conv_state.size(2) == K - 1);
    TORCH_CHECK(slots.scalar_type() == torch::kInt32 && slots.numel() >= rows);
    TORCH_CHECK(y.scalar_type() == torch::kFloat32 && y.is_contiguous() && y.size(0) >= rows && y.size(1) == C);
    LLM_CUDA_CHECK(llm::launch_gdn_conv_step(static_cast<const __nv_bfloat16*>(in.data_ptr()), (int)in.stride(0),
                                             static_cast<const float*>(conv_w.data_ptr()), static_cast<float*>(conv_state.data_ptr()),
                                             static_cast<const int*>(slots.data_ptr()), static_cast<float*>(y.data_ptr()), rows, C, K, cur_stream()));
}

// ... second launch: delta rule on every (row, value head) + gated RMSNorm -> out[rows, n_v * d] bf16
static void gdn_recurrent_step(const Tensor& y, const Tensor& in, int64_t z_off, int64_t ab_off, const Tensor& ssm_a, const Tensor& dt_bias,
                               const Tensor& norm_w, Tensor rec, const Tensor& slots, Tensor out, int64_t n_k, int64_t v_head_offset,
                               double eps) {
    check_cuda(y, "y"); check_cuda(rec, "rec");
    const c10::cuda::CUDAGuard guard(y.device());
    const int rows = (int)in.size(0), n_v = (int)rec.size(1), d = (int)rec.size(2);
    TORCH_CHECK(rec.scalar_type() == torch::kFloat32 && rec.is_contiguous() && rec.dim() == 4 && rec.size(3) == d);
    TORCH_CHECK(y.scalar_type() == torch::kFloat32 && y.is_contiguous() && y.size(0) >= rows && y.size(1) == 2 * n_k * d + n_v * d);
    TORCH_CHECK(in.scalar_type() == torch::kBFloat16 && in.dim() == 2 && in.stride(1) == 1);
    TORCH_CHECK(z_off + n_v * d <= in.size(1) && ab_off + 2 * n_v <= in.size(1));
    TORCH_CHECK(ssm_a.scalar_type() == torch::kFloat32 && ssm_a.numel() == n_v && dt_bias.scalar_type() == torch::kFloat32 && dt_bias.numel() == n_v);
    TORCH_CHECK(norm_w.scalar_type() == torch::kFloat32 && norm_w.numel() == d);
    TORCH_CHECK(slots.scalar_type() == torch::kInt32 && slots.numel() >= rows);
    TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.dim() == 2 && out.stride(1) == 1 && out.size(0) >= rows && out.size(1) >= n_v * d);
    llm::GdnStepParams p{};
    p.y = static_cast<const float*>(y.data_ptr()); p.C = (int)y.size(1);
    p.in = static_cast<const __nv_bfloat16*>(in.data_ptr()); p.in_stride = (int)in.stride(0); p.z_off = (int)z_off; p.ab_off = (int)ab_off;
    p.ssm_a = static_cast<const float*>(ssm_a.data_ptr()); p.dt_bias = static_cast<const float*>(dt_bias.data_ptr());
    p.norm_w = static_cast<const float*>(norm_w.data_ptr());
    p.rec = static_cast<float*>(rec.data_ptr()); p.slots = static_cast<const int*>(slots.data_ptr());
    p.out = static_cast<__nv_bfloat16*>(out.data_ptr()); p.out_stride = (int)out.stride(0);
    p.n_k = (int)n_k; p.n_v = n_v; p.v_head_offset = (int)v_head_offset; p.eps = (float)eps;
    LLM_CUDA_CHECK(llm::launch_gdn_recurrent_step(p, rows, d, cur_stream()));
}

static void attn_decode(const Tensor& q, const Tensor& kv, Tensor out, const Tensor& block_table, const Tensor& seq_lens,
                        const OptTensor& part_o, const OptTensor& part_ml, const OptTensor& tickets, int64_t n_heads,
                        int64_t n_kv_heads, int64_t head_dim, int64_t rows_per_seq, double scale, int64_t n_splits) {
    check_cuda(q, "q");
    const c10::cuda::CUDAGuard guard(q.device());
    const int batch = (int)seq_lens.numel();
    llm::AttnDecodeParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q.data_ptr()); p.kv = static_cast<const __nv_bfloat16*>(kv.data_ptr());
    if (kv.scalar_type() == torch::kUInt8) {
        TORCH_CHECK(kv.dim() == 2, "an 8-bit KV layer is [n_pages, page_bytes]");
        p.kv_q8 = 1; p.page_bytes = (size_t)kv.size(1); p.scale_off = (size_t)2 * n_kv_heads * 64 * head_dim;
        TORCH_CHECK(p.page_bytes == p.scale_off + p.scale_off / 16, "8-bit KV page size does not match heads x head_dim");
    } else {
        TORCH_CHECK(kv.scalar_type() == torch::kBFloat16, "KV cache must be bf16 or 8-bit");
    }
    p.out = static_cast<__nv_bfloat16*>(out.data_ptr());
    p.block_table = static_cast<const int*>(block_table.data_ptr()); p.seq_lens = static_cast<const int*>(seq_lens.data_ptr());
    p.part_o = mptr<float>(part_o); p.part_ml = mptr<float>(part_ml); p.tickets = mptr<unsigned>(tickets);
    p.n_heads = (int)n_heads; p.n_kv_heads = (int)n_kv_heads; p.head_dim = (int)head_dim; p.max_pages = (int)block_table.size(1);
    p.rows_per_seq = (int)rows_per_seq; p.scale = (float)scale;
    p.n_pages = (int)kv.size(0);
    if (n_splits > 1) {
        TORCH_CHECK(part_o.has_value() && part_ml.has_value() && tickets.has_value(), "split decode needs scratch");
        TORCH_CHECK(part_o->numel() >= (int64_t)batch * n_kv_heads * n_splits * 16 * head_dim, "part_o too small");
        TORCH_CHECK(part_ml->numel() >= (int64_t)batch * n_kv_heads * n_splits * 32, "part_ml too small");
        TORCH_CHECK(tickets->numel() >= (int64_t)batch * n_kv_heads, "tickets too small");
    }
    LLM_CUDA_CHECK(llm::launch_attn_decode(p, batch, (int)n_splits, cur_stream()));
}

static void attn_prefill(const Tensor& q, const Tensor& kv, Tensor out, const Tensor& block_table, const Tensor& cu_q,
                         const Tensor& ctx_lens, int64_t n_heads, int64_t n_kv_heads, int64_t head_dim, double scale, int64_t max_q_len,
                         bool tensor_core, const OptTensor& status) {
    check_cuda(q, "q");
    const c10::cuda::CUDAGuard guard(q.device());
    llm::AttnPrefillParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q.data_ptr()); p.kv = static_cast<const __nv_bfloat16*>(kv.data_ptr());
    p.out = static_cast<__nv_bfloat16*>(out.data_ptr());
    p.block_table = static_cast<const int*>(block_table.data_ptr()); p.cu_q = static_cast<const int*>(cu_q.data_ptr());
    p.ctx_lens = static_cast<const int*>(ctx_lens.data_ptr());
    p.n_heads = (int)n_heads; p.n_kv_heads = (int)n_kv_heads; p.head_dim = (int)head_dim; p.max_pages = (int)block_table.size(1);
    p.scale = (float)scale; p.n_pages = (int)kv.size(0);
    if (tensor_core) {
        TORCH_CHECK(head_dim == 128, "the tcgen05 prefill attention is built for head_dim 128");
        LLM_CUDA_CHECK(llm::launch_attn_prefill_tc(p, (int)ctx_lens.numel(), (int)max_q_len, mptr<int>(status), cur_stream()));
    } else {
        LLM_CUDA_CHECK(llm::launch_attn_prefill(p, (int)ctx_lens.numel(), (int)max_q_len, cur_stream()));
    }
}


static void argmax(const Tensor& logits, const OptTensor& tokens, const OptTensor& pairs, int64_t idx_offset) {
    check_cuda(logits, "logits");
    const c10::cuda::CUDAGuard guard(logits.device());
    TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && (tokens.has_value() || pairs.has_value()));
    if (tokens.has_value()) TORCH_CHECK(tokens->scalar_type() == torch::kInt32 && tokens->numel() >= logits.size(0));
    if (pairs.has_value()) TORCH_CHECK(pairs->scalar_type() == torch::kInt32 && pairs->numel() >= 2 * logits.size(0) && pairs->is_contiguous());
    LLM_CUDA_CHECK(llm::launch_argmax(static_cast<const float*>(logits.data_ptr()), (int)logits.size(0), (int)logits.size(1),
                                      (int)logits.stride(0), mptr<int>(tokens), mptr<int>(pairs), (int)idx_offset, cur_stream()));
}

static void argmax_merge(const Tensor& gathered, int64_t ranks, int64_t rows, Tensor tokens) {
    check_cuda(gathered, "gathered");
    const c10::cuda::CUDAGuard guard(gathered.device());
    TORCH_CHECK(gathered.scalar_type() == torch::kInt32 && gathered.is_contiguous() && gathered.numel() >= ranks * rows * 2);
    TORCH_CHECK(tokens.scalar_type() == torch::kInt32 && tokens.numel() >= rows);
    LLM_CUDA_CHECK(llm::launch_argmax_merge(static_cast<const int*>(gathered.data_ptr()), (int)ranks, (int)rows,
                                            static_cast<int*>(tokens.data_ptr()), cur_stream()));
}

static void sample(const Tensor& logits, const Tensor& temperature, const Tensor& top_k, const Tensor& top_p, const Tensor& seeds,
                   const Tensor& step, Tensor tokens, const OptTensor& probs_out) {
    const c10::cuda::CUDAGuard guard(logits.device());
    TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && tokens.scalar_type() == torch::kInt32);
    TORCH_CHECK(seeds.scalar_type() == torch::kInt64 && step.scalar_type() == torch::kInt32 && top_k.scalar_type() == torch::kInt32);
    llm::SampleParams p{};
    p.logits = static_cast<const float*>(logits.data_ptr()); p.rows = (int)logits.size(0); p.vocab = (int)logits.size(1);
    p.stride = (int)logits.stride(0);
    p.temperature = static_cast<const float*>(temperature.data_ptr()); p.top_k = static_cast<const int*>(top_k.data_ptr());
    p.top_p = static_cast<const float*>(top_p.data_ptr()); p.seeds = static_cast<const uint64_t*>(seeds.data_ptr());
    p.step = static_cast<const int*>(step.data_ptr()); p.tokens = static_cast<int*>(tokens.data_ptr());
    p.probs_out = mptr<float>(probs_out);
    LLM_CUDA_CHECK(llm::launch_sample(p, cur_stream()));
}

// pass 1 of sampling over a vocabulary-sharded head: pairs[rows, k, 2] = this shard's k best (float bits, global token id)
static void sample_candidates(const Tensor& logits, int64_t idx_offset, Tensor pairs) {
    const c10::cuda::CUDAGuard guard(logits.device());
    TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && pairs.scalar_type() == torch::kInt32 && pairs.is_contiguous());
    TORCH_CHECK(pairs.dim() == 3 && pairs.size(0) >= logits.size(0) && pairs.size(2) == 2 && pairs.size(1) >= 1 && pairs.size(1) <= 1024);
    llm::SampleParams p{};
    p.logits = static_cast<const float*>(logits.data_ptr()); p.rows = (int)logits.size(0); p.vocab = (int)logits.size(1);
    p.stride = (int)logits.stride(0);
    p.cand_out = static_cast<int*>(pairs.data_ptr()); p.cand_k = (int)pairs.size(1); p.idx_offset = (int)idx_offset;
    LLM_CUDA_CHECK(llm::launch_sample(p, cur_stream()));
}

// pass 2: draw from the all-gathered pairs [ranks, rows, k, 2]
static void sample_merged(const Tensor& gathered, const Tensor& temperature, const Tensor& top_k, const Tensor& top_p, const Tensor& seeds,
                          const Tensor& step, Tensor tokens) {
    const c10::cuda::CUDAGuard guard(gathered.device());
    TORCH_CHECK(gathered.scalar_type() == torch::kInt32 && gathered.is_contiguous() && gathered.dim() == 4 && gathered.size(3) == 2);
    TORCH_CHECK(tokens.scalar_type() == torch::kInt32 && tokens.numel() >= gathered.size(1));
    TORCH_CHECK(seeds.scalar_type() == torch::kInt64 && step.scalar_type() == torch::kInt32 && top_k.scalar_type() == torch::kInt32);
    llm::SampleParams p{};
    p.rows = (int)gathered.size(1); p.vocab = (int)(gathered.size(0) * gathered.size(2));
    p.merge_pairs = static_cast<const int*>(gathered.data_ptr()); p.merge_ranks = (int)gathered.size(0); p.merge_k = (int)gathered.size(2);
    p.temperature = static_cast<const float*>(temperature.data_ptr()); p.top_k = static_cast<const int*>(top_k.data_ptr());
    p.top_p = static_cast<const float*>(top_p.data_ptr()); p.seeds = static_cast<const uint64_t*>(seeds.data_ptr());
    p.step = static_cast<const int*>(step.data_ptr()); p.tokens = static_cast<int*>(tokens.data_ptr());
    LLM_CUDA_CHECK(llm::launch_sample(p, cur_stream()));
}

static void penalties_dense(Tensor logits, const Tensor& counts, const Tensor& presence, const Tensor& frequency) {
    const c10::cuda::CUDAGuard guard(logits.device());
    TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && counts.scalar_type() == torch::kInt16 && logits.dim() == 2 && counts.dim() == 2);
    TORCH_CHECK(counts.size(0) >= logits.size(0) && counts.size(1) >= logits.size(1), "count table smaller than the logits");
    TORCH_CHECK(presence.numel() >= logits.size(0) && frequency.numel() >= logits.size(0));
    LLM_CUDA_CHECK(llm::launch_penalties_dense(static_cast<float*>(logits.data_ptr()), (int)logits.size(0), (int)logits.size(1), (int)logits.stride(0),
                                               static_cast<const unsigned short*>(counts.data_ptr()), (int)counts.stride(0),
                                               static_cast<const float*>(presence.data_ptr()), static_cast<const float*>(frequency.data_ptr()), cur_stream()));
}

static void count_tokens(Tensor counts, const Tensor& tokens, int64_t v0, int64_t vocab) {
    const c10::cuda::CUDAGuard guard(counts.device());
    TORCH_CHECK(counts.scalar_type() == torch::kInt16 && tokens.scalar_type() == torch::kInt32 && counts.dim() == 2);
    TORCH_CHECK(counts.size(0) >= tokens.numel() && counts.size(1) >= vocab);
    LLM_CUDA_CHECK(llm::launch_count_tokens(static_cast<unsigned short*>(counts.data_ptr()), (int)counts.stride(0),
                                            static_cast<const int*>(tokens.data_ptr()), (int)v0, (int)vocab, (int)tokens.numel(), cur_stream()));
}

static void nan_scan(const Tensor& x, Tensor counts) {
    const c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.is_contiguous() && counts.scalar_type() == torch::kInt32 && counts.numel() >= 2);
    const int dt = x.scalar_type() == torch::kFloat32 ? 0 : 1;
    TORCH_CHECK(dt == 0 || x.scalar_type() == torch::kBFloat16, "nan_scan: fp32 or bf16 only");
    LLM_CUDA_CHECK(llm::launch_nan_scan(x.data_ptr(), (size_t)x.numel(), dt, static_cast<int*>(counts.data_ptr()), cur_stream()));
}

static void spec_verify_greedy(const Tensor& draft, const Tensor& target, Tensor n_accept, Tensor out_tokens) {
    const c10::cuda::CUDAGuard guard(draft.device());
    TORCH_CHECK(draft.scalar_type() == torch::kInt32 && target.scalar_type() == torch::kInt32);
    LLM_CUDA_CHECK(llm::launch_spec_verify_greedy(static_cast<const int*>(draft.data_ptr()), static_cast<const int*>(target.data_ptr()),
                                                  (int)draft.size(0), (int)draft.size(1), static_cast<int*>(n_accept.data_ptr()),
                                                  static_cast<int*>(out_tokens.data_ptr()), cur_stream()));
}

static void spec_verify_reject(const Tensor& p_target, const Tensor& p_draft, const Tensor& draft, const Tensor& seeds, const Tensor& step,
                               Tensor n_accept, Tensor out_tokens) {
    const c10::cuda::CUDAGuard guard(draft.device());
    TORCH_CHECK(p_target.is_contiguous() && p_draft.is_contiguous() && draft.is_contiguous());
    llm::SpecRejectParams p{};
    p.p_target = static_cast<const float*>(p_target.data_ptr()); p.p_draft = static_cast<const float*>(p_draft.data_ptr());
    p.draft = static_cast<const int*>(draft.data_ptr()); p.seeds = static_cast<const uint64_t*>(seeds.data_ptr());
    p.step = static_cast<const int*>(step.data_ptr());
    p.batch = (int)draft.size(0); p.depth = (int)draft.size(1); p.vocab = (int)p_target.size(-1);
    p.n_accept = static_cast<int*>(n_accept.data_ptr()); p.out_tokens = static_cast<int*>(out_tokens.data_ptr());
    LLM_CUDA_CHECK(llm::launch_spec_verify_reject(p, cur_stream()));
}

static void moe_topk(const Tensor& logits, int64_t k, bool renorm, Tensor ids, Tensor weights, const OptTensor& counts) {
    const c10::cuda::CUDAGuard guard(logits.device());
    TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && logits.is_contiguous());
    LLM_CUDA_CHECK(llm::launch_moe_topk(static_cast<const float*>(logits.data_ptr()), (int)logits.size(0), (int)logits.size(1), (int)k,
                                        renorm ? 1 : 0, static_cast<int*>(ids.data_ptr()), static_cast<float*>(weights.data_ptr()),
                                        mptr<int>(counts), cur_stream()));
}

// tensor-core GEMM: out[M, N] (+)= x[M, K] * dequant(W)[N, K]^T
static void gemm_tc(const Tensor& w, int64_t fmt, int64_t n, int64_t k, const Tensor& x, Tensor out, int64_t epi, const OptTensor& bias,
                    const OptTensor& accum, const OptTensor& tickets, int64_t ksplit, const OptTensor& status, int64_t debug_ptr, int64_t flags, const OptTensor& tp,
                    const OptTensor& partials) {
    check_cuda(w, "w"); check_cuda(x, "x"); check_cuda(out, "out");
    const c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && x.is_contiguous(), "gemm_tc input must be contiguous bf16");
    llm::GemmTcParams p{};
    p.w = static_cast<const uint8_t*>(w.data_ptr()); p.fmt = (int)fmt; p.n = (int)n; p.k = (int)k; p.m = (int)x.size(0);
    p.x = static_cast<const __nv_bfloat16*>(x.data_ptr());
    p.out = out.data_ptr(); p.out_stride = (int)out.stride(0); p.out_f32 = out.scalar_type() == torch::kFloat32;
    p.epi = (int)epi; p.bias = cptr<float>(bias); p.status = mptr<int>(status);
    p.accum = mptr<float>(accum); p.tickets = mptr<unsigned>(tickets); p.ksplit = (int)ksplit;
    if (partials.has_value() && partials->numel() >= 148 * 2 * 128 * 32 && partials->scalar_type() == torch::kFloat32) p.partials = mptr<float>(partials);
    p.debug = reinterpret_cast<int*>(debug_ptr); p.flags = (int)flags;
    p.tp = tp.has_value() ? reinterpret_cast<const llm::TpFuse*>(tp->data_ptr()) : nullptr;
    if (tp.has_value()) TORCH_CHECK(p.m <= 32 && epi == llm::EPI_RESID, "fused tensor-parallel epilogue: residual mode, at most 32 rows");
    p.accum_stride = accum.has_value() ? (int)accum->stride(0) : 0;
    if (epi == llm::EPI_RESID) TORCH_CHECK(p.out_f32, "residual epilogue updates an fp32 stream");
    if (accum.has_value()) {
        int bm = 0, ks = 0;
        llm::gemm_tc_plan(p.m, p.n, p.k, p.ksplit, &bm, &ks);
        const int64_t n_tiles = (n + 127) / 128, m_tiles = (p.m + bm - 1) / bm;
        TORCH_CHECK(ks == 1 || (accum->size(0) >= p.m && accum->stride(0) >= n_tiles * 128), "split-K scratch too small");
        TORCH_CHECK(ks == 1 || (tickets.has_value() && tickets->numel() >= n_tiles * m_tiles), "ticket scratch too small");
    }
    LLM_CUDA_CHECK(llm::launch_gemm_tc(p, cur_stream()));
}

// Column-parallel GEMM whose activation rows are all-gathered from the ranks inside the launch (AgFuse in gemm_tc.h).
// `desc` is a host int64 tensor: [src ptr x8, avail ptr x8, stage ptr, staged ptr, world, rank, rows_per_rank, copy_ctas, epoch, spin_limit].
static void gemm_tc_allgather(const Tensor& w, int64_t fmt, int64_t n, int64_t k, int64_t m, Tensor out, int64_t epi, const OptTensor& bias,
                              const OptTensor& status, const Tensor& desc) {
    check_cuda(w, "w"); check_cuda(out, "out");
    const c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(desc.device().is_cpu() && desc.scalar_type() == torch::kInt64 && desc.numel() >= 24);
    const int64_t* d = desc.data_ptr<int64_t>();
    llm::GemmTcParams p{};
    p.w = static_cast<const uint8_t*>(w.data_ptr()); p.fmt = (int)fmt; p.n = (int)n; p.k = (int)k; p.m = (int)m;
    p.x = nullptr;
    p.out = out.data_ptr(); p.out_stride = (int)out.stride(0); p.out_f32 = out.scalar_type() == torch::kFloat32;
    p.epi = (int)epi; p.bias = cptr<float>(bias); p.status = mptr<int>(status);
    p.ksplit = 1;
    p.ag_on = 1;
    for (int i = 0; i < 8; ++i) {
        p.ag.src[i] = reinterpret_cast<const __nv_bfloat16*>(d[i]);
        p.ag.avail[i] = reinterpret_cast<unsigned*>(d[8 + i]);
    }
    p.ag.stage = reinterpret_cast<__nv_bfloat16*>(d[16]);
    p.ag.staged = reinterpret_cast<unsigned*>(d[17]);
    p.ag.world = (int)d[18]; p.ag.rank = (int)d[19]; p.ag.rows_per_rank = (int)d[20]; p.ag.copy_ctas = (int)d[21];
    p.ag.epoch = (unsigned)d[22]; p.ag.spin_limit = (unsigned)d[23];
    TORCH_CHECK(m <= (int64_t)p.ag.world * p.ag.rows_per_rank, "more rows than the ranks hold");
    if (epi == llm::EPI_RESID) TORCH_CHECK(p.out_f32, "residual epilogue updates an fp32 stream");
    LLM_CUDA_CHECK(llm::launch_gemm_tc(p, cur_stream()));
}

// Row-parallel GEMM whose partial tiles are reduce-scattered to the owners of their rows inside the launch (RsFuse in gemm_tc.h).
// `desc` is a host int64 tensor: [inbox ptr x8, flags ptr x8, world, rank, rows_per_rank, n_cap, parity, flags_per_parity].
static void gemm_tc_rs(const Tensor& w, int64_t fmt, int64_t n, int64_t k, const Tensor& x, const OptTensor& status, const Tensor& desc) {
    check_cuda(w, "w"); check_cuda(x, "x");
    const c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && x.is_contiguous(), "gemm_tc_rs input must be contiguous bf16");
    TORCH_CHECK(desc.device().is_cpu() && desc.scalar_type() == torch::kInt64 && desc.numel() >= 22);
    const int64_t* d = desc.data_ptr<int64_t>();
    llm::GemmTcParams p{};
    p.w = static_cast<const uint8_t*>(w.data_ptr()); p.fmt = (int)fmt; p.n = (int)n; p.k = (int)k; p.m = (int)x.size(0);
    p.x = static_cast<const __nv_bfloat16*>(x.data_ptr());
    p.out = nullptr; p.epi = llm::EPI_STORE; p.status = mptr<int>(status); p.ksplit = 1;
    p.rs_on = 1;
    for (int i = 0; i < 8; ++i) {
        p.rs.inbox[i] = reinterpret_cast<__nv_bfloat16*>(d[i]);
        p.rs.flags[i] = reinterpret_cast<unsigned*>(d[8 + i]);
    }
    p.rs.world = (int)d[16]; p.rs.rank = (int)d[17]; p.rs.rows_per_rank = (int)d[18]; p.rs.n_cap = (int)d[19];
    p.rs.parity = (int)d[20]; p.rs.flags_per_parity = (int)d[21];
    TORCH_CHECK(p.rs.world >= 1 && p.rs.world <= 8 && p.rs.rank >= 0 && p.rs.rank < p.rs.world, "bad reduce-scatter group");
    TORCH_CHECK(p.m <= (int64_t)p.rs.world * p.rs.rows_per_rank, "more rows than the ranks own");
    TORCH_CHECK(n <= p.rs.n_cap && p.rs.n_cap % 8 == 0, "inbox rows narrower than the output");
    for (int i = 0; i < p.rs.world; ++i) TORCH_CHECK(p.rs.inbox[i] && p.rs.flags[i], "null inbox / flags pointer");
    TORCH_CHECK((p.rs.rows_per_rank / llm::gemm_tc_rs_block_m(p.m, p.rs.rows_per_rank)) <= p.rs.flags_per_parity, "too few arrival counters");
    LLM_CUDA_CHECK(llm::launch_gemm_tc(p, cur_stream()));
}

static void rs_reduce_norm(int64_t inbox_ptr, int64_t flags_ptr, int64_t target, int64_t world, int64_t rows_per_rank, int64_t n_cap,
                           int64_t block_m, Tensor h, const OptTensor& norm_w, const OptTensor& xn, double eps, int64_t spin_limit,
                           const OptTensor& status) {
    check_cuda(h, "h");
    const c10::cuda::CUDAGuard guard(h.device());
    TORCH_CHECK(h.scalar_type() == torch::kFloat32 && h.is_contiguous() && h.dim() == 2, "h must be contiguous fp32 [rows, d]");
    TORCH_CHECK(inbox_ptr != 0 && flags_ptr != 0, "null inbox / flags pointer");
    TORCH_CHECK(h.size(1) <= n_cap, "inbox rows narrower than h");
    if (norm_w.has_value()) {
        TORCH_CHECK(xn.has_value() && xn->scalar_type() == torch::kBFloat16 && xn->is_contiguous() && xn->size(0) >= h.size(0) && xn->size(1) == h.size(1));
        TORCH_CHECK(norm_w->scalar_type() == torch::kFloat32 && norm_w->numel() == h.size(1));
    }
    LLM_CUDA_CHECK(llm::launch_rs_reduce_norm(reinterpret_cast<const __nv_bfloat16*>(inbox_ptr), reinterpret_cast<const unsigned*>(flags_ptr),
                                              (unsigned)target, (int)world, (int)rows_per_rank, (int)n_cap, (int)block_m,
                                              static_cast<float*>(h.data_ptr()), cptr<float>(norm_w),
                                              xn.has_value() ? static_cast<__nv_bfloat16*>(xn->data_ptr()) : nullptr, (int)h.size(0), (int)h.size(1),
                                              (float)eps, (unsigned)spin_limit, mptr<int>(status), cur_stream()));
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("set_pdl", [](bool on) { llm::pdl_enabled() = on; });
    m.def("bounds_status", [](bool reset) { return llm::bounds_status_ops(reset) | llm::bounds_status_attention(reset) | llm::bounds_status_attention_tc(reset); });
#ifdef LLM_BOUNDS_CHECK
    m.attr("bounds_check_build") = true;
#else
    m.attr("bounds_check_build") = false;
#endif
    m.def("gemv", &gemv);
    m.def("kv_dequant_pages", &kv_dequant_pages);
    m.def("gdn_conv_step", &gdn_conv_step);
    m.def("gdn_recurrent_step", &gdn_recurrent_step);
    m.def("moe_route", &moe_route);
    m.def("moe_gemv", &moe_gemv);
    m.def("moe_route_only", &moe_route_only);
    m.def("moe_combine_sorted", &moe_combine_sorted);
    m.def("gemm_tc_grouped", &gemm_tc_grouped);
    m.def("gemm_tc", &gemm_tc);
    m.def("gemm_tc_allgather", &gemm_tc_allgather);
    m.def("gemm_tc_rs", &gemm_tc_rs);
    m.def("rs_reduce_norm", &rs_reduce_norm);
    m.def("gemm_tc_rs_block_m", [](int64_t m_, int64_t rows_per_rank) { return (int64_t)llm::gemm_tc_rs_block_m((int)m_, (int)rows_per_rank); });
    m.def("dequant", &dequant);
    m.def("gather_rows", &gather_rows);
    m.def("rmsnorm", &rmsnorm);
    m.def("mtp_concat_norm", &mtp_concat_norm);
    m.def("rope_kv", &rope_kv);
    m.def("attn_decode", &attn_decode);
    m.def("attn_prefill", &attn_prefill);
    m.def("argmax", &argmax);
    m.def("argmax_merge", &argmax_merge);
    m.def("sample", &sample);
    m.def("sample_candidates", &sample_candidates);
    m.def("sample_merged", &sample_merged);
    m.def("penalties_dense", &penalties_dense);
    m.def("count_tokens", &count_tokens);
    m.def("nan_scan", &nan_scan);
    m.def("spec_verify_greedy", &spec_verify_greedy);
    m.def("spec_verify_reject", &spec_verify_reject);
    m.def("moe_topk", &moe_topk);
    m.def("attn_decode_pick_splits", &llm::attn_decode_pick_splits);
    m.def("gemv_pick_ksplit", &llm::gemv_pick_ksplit);
}
