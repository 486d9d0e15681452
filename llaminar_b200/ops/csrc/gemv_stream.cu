// Streaming GEMV for decode at batch 1..4:  out[m, n] = sum_k x[m, k] * W[n, k], M <= 4 rows, straight from quantised chunks.
//
// Same arithmetic as gemv.cu (lane == weight row, int8 activations quantised in the prologue, dp4a), different plumbing:
//   * persistent CTAs, one per SM, each streaming a contiguous range of (tile, chunk) work ("stream-K"), so every SM moves the
//     same number of bytes whatever the matrix shape;
//   * the packed chunks arrive by bulk copy (cp.async.bulk, one per 128 x 256 chunk) in a ring of shared-memory slots filled
//     by one elected producer thread; weights are constants, so under programmatic dependent launch the ring is filled before
//     the wait for the previous kernel.  Measured on a bare ring of this shape: 6.9 TB/s, against 3.4-3.9 TB/s for the
//     register-path kernel whose warps each keep one chunk of loads in flight;
//   * sixteen compute warps: warp (g, q) owns rows 32 g .. 32 g + 31 of the tile and every fourth chunk (q = chunk mod 4), so a
//     warp revisits a ring slot exactly once per revolution (the ring has a multiple of four slots) and 1-bit mbarrier
//     parities stay exact;
//   * a tile split between CTAs is finished by the CTA that holds its first chunk; the others park their partial sums in
//     per-CTA slots and bump the tile's counter.  The sum runs in CTA order: results do not depend on timing.
// Epilogues: store (bf16 / fp32, + bias), residual add into the fp32 stream, SwiGLU over paired gate / up rows.  Grouped expert
// work, per-slot expert matrices and the fused tensor-parallel epilogue stay with gemv.cu.
//
// Replaces, with gemv.cu, the reference's nativeVnniGemv_* family (reference: src/v2/kernels/cuda/gemm/CUDANativeVNNIGemvTuned.cu:332-1672).
#include <cuda.h>

#include "formats.cuh"
#include "launch.h"
#include "gemv.h"
#include "tc_common.cuh"

namespace llm {
namespace gs {
using namespace tc5;

constexpr int N_WARPS = 16;                    // compute warps
constexpr int THREADS = (N_WARPS + 1) * 32;    // + the producer warp
constexpr int N_COMPUTE = N_WARPS * 32;
constexpr uint32_t TICKET_SPIN = 1u << 20;

struct Extra {
    float* partials;           // [grid][4][128] partial sums parked by the CTAs that do not finish a split tile
    unsigned* tickets;         // [n_tiles] arrivals at a split tile, zero between launches
    int* status;               // STATUS_TIMEOUT is written here when a bounded wait gives up
    int slots;                 // ring slots (4 or 8)
    int act_cap;               // activation blocks kept per row
};

LLM_DEVICE void bar_compute() { asm volatile("bar.sync 1, %0;" ::"n"(N_COMPUTE) : "memory"); }
LLM_DEVICE void bar_rows() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// The flattened (tile, chunk) range of CTA b and its walk, unit by unit (a unit = the part of one tile inside the range).
struct Unit { int tile, kb0, nkb, first_cta, last_cta; };
struct Walk {
    int k_blocks, total, G, pos, end;
    LLM_DEVICE void init(int kb, int n_tiles, int grid, int cta) {
        k_blocks = kb; total = kb * n_tiles; G = grid;
        pos = (int)(((unsigned)cta * (unsigned)total) / (unsigned)G);
        end = (int)(((unsigned)(cta + 1) * (unsigned)total) / (unsigned)G);
    }
    // 32-bit arithmetic: the launcher refuses problems with (chunks + 1) * grid >= 2^32
    LLM_DEVICE int cta_of(int x) const { return (int)(((unsigned)(x + 1) * (unsigned)G - 1u) / (unsigned)total); }
    LLM_DEVICE bool next(Unit& u) {
        if (pos >= end) return false;
        u.tile = pos / k_blocks;
        u.kb0 = pos - u.tile * k_blocks;
        u.nkb = min(k_blocks - u.kb0, end - pos);
        u.first_cta = cta_of(u.tile * k_blocks);
        u.last_cta = cta_of(u.tile * k_blocks + k_blocks - 1);
        pos += u.nkb;
        return true;
    }
};

// RMSNorm (optional) + int8 quantisation of the activation blocks this CTA will meet: blocks kb_first, kb_first + 1, ...
// (mod k_blocks), n_act of them, kept at acts[m * act_cap + i].  Run by the 512 compute threads.
template <int M, int NORM>
LLM_DEVICE void quantise_acts(const GemvParams& p, int kb_first, int n_act, int act_cap, ActBlk* acts, float* s_red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float rms[M];
    // One activation row with a fused RMSNorm (decode at batch 1): the values this CTA will quantise and their gains are
    // loaded together with the full-row pass, before the reduction, and stay in registers across it, so the prologue has one
    // memory round trip on its critical path instead of two.
    constexpr int QPT = 4;                      // quads a thread may keep
    const int n_quads_all = n_act * 64;
    const bool in_regs = NORM && M == 1 && n_quads_all <= QPT * N_COMPUTE;
    float4 keep_v[QPT], keep_g[QPT];
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < QPT; ++j) {
            const int qd = tid + j * N_COMPUTE;
            if (qd < n_quads_all) {
                int kb = kb_first + (qd >> 6);
                if (kb >= p.k_blocks) kb -= p.k_blocks;
                const int col = kb * 256 + (qd & 63) * 4;
                keep_v[j] = *reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + col);
                keep_g[j] = *reinterpret_cast<const float4*>(p.norm_w + col);
            }
        }
    }
    if (NORM) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float ss = 0.f;
            const float4* x4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + (size_t)m * p.x_stride);
            for (int i = tid; i < p.k / 4; i += N_COMPUTE) {
                const float4 v = x4[i];
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            ss = warp_sum(ss);
            if (lane == 0) s_red[warp * M + m] = ss;
        }
        bar_compute();
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float t = 0.f;
            for (int w = 0; w < N_WARPS; ++w) t += s_red[w * M + m];
            rms[m] = rsqrtf(t / p.k + p.eps);
        }
        bar_compute();                          // s_red is reused by the main loop
    }
    const int n_quads = n_act * 64;             // 4 consecutive columns per thread, 8 threads per 32-column block
    // quantise one quad (its 32-column block is shared by 8 neighbouring lanes) and store it
    auto emit = [&](int m, int qd, float v0, float v1, float v2, float v3) {
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
        ActBlk& ab = acts[m * act_cap + (qd >> 6)];
        const int qi = qd & 63;
        ab.a[qi] = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | ((q3 & 0xff) << 24);
        if ((qi & 7) == 0) ab.d[qi >> 3] = d;
        if ((qi & 3) == 0) ab.ds16[qi >> 2] = d * s;
    };
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < QPT; ++j) {
            const int qd = tid + j * N_COMPUTE;  // whole warps are in or out: n_quads is a multiple of 64
            if (qd < n_quads) {
                const float4 v = keep_v[j], g = keep_g[j];
                emit(0, qd, v.x * rms[0] * g.x, v.y * rms[0] * g.y, v.z * rms[0] * g.z, v.w * rms[0] * g.w);
            }
        }
    } else {
        for (int m = 0; m < M; ++m) {
            for (int qd = tid; qd < n_quads; qd += N_COMPUTE) {
                int kb = kb_first + (qd >> 6);
                if (kb >= p.k_blocks) kb -= p.k_blocks;
                const int col = kb * 256 + (qd & 63) * 4;
                if (NORM) {
                    const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + (size_t)m * p.x_stride + col);
                    const float4 g = *reinterpret_cast<const float4*>(p.norm_w + col);
                    emit(m, qd, v.x * rms[m] * g.x, v.y * rms[m] * g.y, v.z * rms[m] * g.z, v.w * rms[m] * g.w);
                } else {
                    const uint2 v = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.x) + (size_t)m * p.x_stride + col);
                    emit(m, qd, bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
                }
            }
        }
    }
    bar_compute();
}

template <int FMT, int M, int NORM>
__global__ void __launch_bounds__(THREADS, 1) gemv_stream_kernel(const GemvParams p, const Extra e) {
    constexpr int CHUNK = FmtTraits<FMT>::CHUNK;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t s_full[8], s_empty[8];
    __shared__ int s_abort[2], s_flag, s_go[2];

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R = e.slots;
    uint8_t* ring = smem;                                                        // R slots of CHUNK bytes
    ActBlk* acts = reinterpret_cast<ActBlk*>(smem + (size_t)R * CHUNK);          // [M][act_cap]
    float* s_red = reinterpret_cast<float*>(acts + (size_t)M * e.act_cap);       // [2][4][M][128]
    uint32_t* s_grid = reinterpret_cast<uint32_t*>(s_red + 2 * 4 * M * 128);     // IQ3_S only
    const uint32_t full_bar = smem_u32(s_full), empty_bar = smem_u32(s_empty), ring_addr = smem_u32(ring);

    if (tid == 0) {
        s_abort[0] = 0; s_abort[1] = 0;
        for (int s = 0; s < R; ++s) { mbar_init(full_bar + s * 8, 1); mbar_init(empty_bar + s * 8, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (FMT == FMT_IQ3_S) {
        for (int i = tid; i < 512; i += THREADS) s_grid[i] = g_iq3s_grid[i];
    }
    __syncthreads();
    volatile int* abort_flag = s_abort;
    Walk it;
    it.init(p.k_blocks, p.n_tiles, gridDim.x, blockIdx.x);
    Unit u;

    if (warp == N_WARPS) {
        // ---------------- producer: one bulk copy per chunk; the first R need no wait and start before the previous kernel ends ----------------
        if (elect_one()) {
            int cc = 0;
            bool ok = true;
            while (ok && it.next(u)) {
                const uint8_t* src = p.w + ((size_t)u.tile * p.k_blocks + u.kb0) * CHUNK;
                for (int c = 0; c < u.nkb && ok; ++c, ++cc) {
                    const int slot = cc % R, phase = (cc / R) & 1;
                    if (cc == R) pdl_wait();
                    ok = mbar_wait(empty_bar + slot * 8, phase ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full_bar + slot * 8, CHUNK);
                    bulk_load(ring_addr + slot * CHUNK, src + (size_t)c * CHUNK, CHUNK, full_bar + slot * 8);
                }
            }
        }
    } else {
        // ---------------- compute warps ----------------
        pdl_wait();
        const int g = warp & 3, q = warp >> 2;
        const int kb_first = it.pos % p.k_blocks;
        const int n_act = min(p.k_blocks, it.end - it.pos);
        quantise_acts<M, NORM>(p, kb_first, n_act, e.act_cap, acts, s_red);
        const int act_stride = e.act_cap * (int)sizeof(ActBlk);
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        int cc = 0, ui = 0;
        bool ok = true;
        // A wait that gives up sets the CTA's abort flag; from then on this warp skips the work but still walks the units, because
        // the named barriers below have no time limit of their own and every compute warp has to reach them.
        while (it.next(u)) {
            for (int c = 0; c < u.nkb; ++c, ++cc) {
                if ((cc & 3) != q || !ok) continue;
                const int slot = cc % R, phase = (cc / R) & 1;
                ok = mbar_wait_warp(full_bar + slot * 8, phase, abort_flag);
                if (!ok) continue;
                int ai = u.kb0 + c - kb_first;
                if (ai < 0) ai += p.k_blocks;
                const uint8_t* chunk = ring + (size_t)slot * CHUNK;
                if constexpr (FMT == FMT_IQ3_S) DotBlock<FMT, M, LdShared>::run(chunk, g, lane, acts + ai, act_stride, acc, s_grid);
                else DotBlock<FMT, M, LdShared>::run(chunk, g, lane, acts + ai, act_stride, acc);
                __syncwarp();                                        // every lane has its bytes in registers
                mbar_arrive_if(empty_bar + slot * 8, lane == 0);
            }
            // ---- the unit is done: add up the four chunk phases of every row ----
            float* red = s_red + (ui & 1) * (4 * M * 128);
            const int r = g * 32 + lane;
#pragma unroll
            for (int m = 0; m < M; ++m) { red[(q * M + m) * 128 + r] = acc[m]; acc[m] = 0.f; }
            if (tid == 0) s_go[ui & 1] = abort_flag[0] ? 0 : 1;       // one reading of the flag for all row threads (they meet at barriers below)
            bar_compute();
            const bool go = s_go[ui & 1] != 0;
            ++ui;
            if (tid >= 128 || !go) continue;
            float v[M];
#pragma unroll
            for (int m = 0; m < M; ++m) v[m] = red[m * 128 + tid] + red[(M + m) * 128 + tid] + red[(2 * M + m) * 128 + tid] + red[(3 * M + m) * 128 + tid];
            const int row = u.tile * 128 + tid;
            if (u.first_cta != u.last_cta) {
                if ((int)blockIdx.x != u.first_cta) {
                    // park and tell the finisher (every thread's stores, then one release from thread 0)
                    float* mine = e.partials + (size_t)blockIdx.x * (4 * 128);
#pragma unroll
                    for (int m = 0; m < M; ++m) __stcg(&mine[m * 128 + tid], v[m]);
                    __threadfence();
                    bar_rows();
                    if (tid == 0) red_release_gpu_add(&e.tickets[u.tile], 1u);
                    continue;
                }
                // finisher: the others hold later chunks of the tile but reach them at the START of their ranges, so they are
                // usually long done; wait (bounded) for their count, then add their slots in CTA order
                const unsigned want = (unsigned)(u.last_cta - u.first_cta);
                if (tid == 0) {
                    int got = 0;
                    for (uint32_t i = 0; i < TICKET_SPIN; ++i) {
                        if (ld_acquire_gpu(&e.tickets[u.tile]) >= want) { got = 1; break; }
                        if (i > 64) { if (abort_flag[0]) break; __nanosleep(64); }
                    }
                    if (!got) abort_flag[0] = 1;
                    s_flag = got;
                }
                bar_rows();
                const bool got = s_flag != 0;
                if (got) for (int cta = u.first_cta + 1; cta <= u.last_cta; ++cta) {
                    const float* theirs = e.partials + (size_t)cta * (4 * 128);
#pragma unroll
                    for (int m = 0; m < M; ++m) v[m] += __ldcg(&theirs[m * 128 + tid]);
                }
                bar_rows();                                          // everybody has read the count's verdict and the slots
                if (tid == 0) e.tickets[u.tile] = 0u;
                if (!got) continue;
            }
            // ---- epilogue of a finished tile ----
            if (p.epi == EPI_SWIGLU) {
                // a 32-row group holds 16 gate rows followed by the 16 matching up rows: pair lanes l and l + 16
                const int col = u.tile * 64 + (tid >> 5) * 16 + (lane & 15);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float other = __shfl_xor_sync(0xffffffffu, v[m], 16);
                    if (lane < 16 && col < p.n / 2)
                        static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.out_stride + col] = __float2bfloat16(silu(v[m]) * other);
                }
            } else if (row < p.n) {
                const float b = p.bias ? p.bias[row] : 0.f;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const size_t idx = (size_t)m * p.out_stride + row;
                    const float o = v[m] + b;
                    if (p.epi == EPI_RESID) static_cast<float*>(p.out)[idx] += o;
                    else if (p.out_f32) static_cast<float*>(p.out)[idx] = o;
                    else static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16(o);
                }
            }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0 && e.status) atomicExch(e.status, (int)STATUS_TIMEOUT);
        for (int i = 0; i < 2000; ++i) __nanosleep(100);      // let bulk copies still in flight land before the shared memory is handed on
    }
}

static size_t smem_bytes(int chunk, int slots, int m, int act_cap) {
    return (size_t)slots * chunk + (size_t)m * act_cap * sizeof(ActBlk) + 2 * 4 * (size_t)m * 128 * sizeof(float) + 512 * sizeof(uint32_t);
}

template <int FMT, int M, int NORM>
static cudaError_t launch_k(const GemvParams& p, const Extra& e, int grid, size_t smem, cudaStream_t st) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t err = cudaFuncSetAttribute(gemv_stream_kernel<FMT, M, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (err != cudaSuccess) return err;
        attr_set = true;
    }
    return launch_pdl(gemv_stream_kernel<FMT, M, NORM>, dim3(grid), dim3(THREADS), smem, st, p, e);
}
template <int FMT, int M>
static cudaError_t launch_m(const GemvParams& p, const Extra& e, int grid, size_t smem, cudaStream_t st) {
    return p.norm_w ? launch_k<FMT, M, 1>(p, e, grid, smem, st) : launch_k<FMT, M, 0>(p, e, grid, smem, st);
}
template <int FMT>
static cudaError_t launch_f(const GemvParams& p, int m, int grid, int chunks_per_cta, float* partials, unsigned* tickets, int* status,
                            cudaStream_t st) {
    constexpr int CHUNK = FmtTraits<FMT>::CHUNK;
    Extra e{partials, tickets, status, 0, 0};
    e.act_cap = p.k_blocks < chunks_per_cta ? p.k_blocks : chunks_per_cta;
    e.slots = 8;
    size_t smem = smem_bytes(CHUNK, 8, m, e.act_cap);
    if (smem > 216 * 1024) { e.slots = 4; smem = smem_bytes(CHUNK, 4, m, e.act_cap); }
    if (smem > 216 * 1024) return cudaErrorNotSupported;
    switch (m) {
        case 1: return launch_m<FMT, 1>(p, e, grid, smem, st);
        case 2: return launch_m<FMT, 2>(p, e, grid, smem, st);
        case 3: return launch_m<FMT, 3>(p, e, grid, smem, st);
        case 4: return launch_m<FMT, 4>(p, e, grid, smem, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace gs

// cudaErrorNotSupported: the call is not one this kernel takes (the caller falls back to launch_gemv).
cudaError_t launch_gemv_stream(const GemvParams& p, int m, float* partials, size_t partials_floats, unsigned* tickets, int* status, cudaStream_t st) {
    if (m < 1 || m > 4 || p.items || p.expert_ids || p.tp || !partials || !tickets) return cudaErrorNotSupported;
    if (p.epi != EPI_STORE && p.epi != EPI_RESID && p.epi != EPI_SWIGLU) return cudaErrorNotSupported;
    if (reinterpret_cast<uintptr_t>(p.w) & 15) return cudaErrorNotSupported;
    const int total = p.n_tiles * p.k_blocks;
    if ((unsigned long long)((long long)total + 1) * 148ull >= (1ull << 32)) return cudaErrorNotSupported;      // 32-bit work indices
    static int cached_sms = 0;
    if (!cached_sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&cached_sms, cudaDevAttrMultiProcessorCount, dev); }
    const int sms = cached_sms > 0 ? cached_sms : 148;
    int grid = total / 4;                       // at least four chunks per CTA: the start-up and the epilogue cost a few chunks' time
    if (grid > sms) grid = sms;
    if (grid < 1) grid = 1;
    if ((size_t)grid * 4 * 128 > partials_floats) return cudaErrorNotSupported;
    const int chunks_per_cta = (total + grid - 1) / grid + 1;
    switch (p.fmt) {
        case FMT_Q4_K: return gs::launch_f<FMT_Q4_K>(p, m, grid, chunks_per_cta, partials, tickets, status, st);
        case FMT_Q5_K: return gs::launch_f<FMT_Q5_K>(p, m, grid, chunks_per_cta, partials, tickets, status, st);
        case FMT_Q6_K: return gs::launch_f<FMT_Q6_K>(p, m, grid, chunks_per_cta, partials, tickets, status, st);
        case FMT_Q8_0: return gs::launch_f<FMT_Q8_0>(p, m, grid, chunks_per_cta, partials, tickets, status, st);
        case FMT_Q4_0: return gs::launch_f<FMT_Q4_0>(p, m, grid, chunks_per_cta, partials, tickets, status, st);
        case FMT_IQ3_S: return gs::launch_f<FMT_IQ3_S>(p, m, grid, chunks_per_cta, partials, tickets, status, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace llm
