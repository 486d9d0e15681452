// out[M, N] = x[M, K] * dequant(W)[N, K]^T on the 5th-generation tensor cores, weights decoded in the main loop.
//
// Roles inside one CTA (320 threads):
//   warps 0-7  dequant producers: lane == weight row; each warp owns a 32-row group and every other
//              256-column chunk (warps 0-3 and 4-7 form two sets, each with its own half of the ring).  Packed bytes go global -> registers (next chunk prefetched), are
//              converted to bf16 and stored into the 128B-swizzled K-major operand tile of the ring
//              stage, one 64-column "atom" (16 KB) at a time.  Afterwards they run the epilogue.
//   warp 8     TMA producer: the activation tile (BM tokens x 64 columns) of each atom, SWIZZLE_128B.
//   warp 9     allocates TMEM, issues tcgen05.mma (A = weights, 128 rows; B = activations, BM columns),
//              releases ring stages with tcgen05.commit.
// The accumulator is D[n, m] in TMEM (128 lanes x BM fp32 columns): weights sit in the MMA M dimension
// so a batch-32 decode step wastes nothing, and the same kernel serves prefill with BM = 256.
// Skinny problems add split-K over blockIdx.z (fp32 atomics into scratch, last CTA runs the epilogue).
// Every mbarrier wait is bounded; on a timeout the kernel raises the status word and tears down cleanly.
//
// Replaces nativeVnniTC_BK64/BK256 + splitk_reduce/streamk_* (mma.sync int8 with in-smem dequant) of the
// reference: src/v2/kernels/cuda/gemm/CUDANativeVNNIPrefillKernels.cu:141-3219.
#include <cuda.h>

#include "formats.cuh"
#include "gemm_tc.h"
#include "tc_common.cuh"
#include "tp_fuse.cuh"
#include "gemv.h"

namespace llm {

namespace tc {
using namespace tc5;

constexpr int A_ATOM_BYTES = 128 * 128;          // 128 weight rows x 64 bf16
constexpr uint32_t SPIN_LIMIT = 1u << 22;

// Bounded waits: tc_common.cuh (mbar_wait for one lane, mbar_wait_warp for a converged warp).  abort_flag[1] is set while the
// TMA lane is inside its own bounded wait for staged rows (fused all-gather): the rest of the pipeline is legitimately stalled.
template <int BM> struct Cfg {
    static constexpr int B_ATOM_BYTES = BM * 128;
    static constexpr int STAGE_BYTES = A_ATOM_BYTES + B_ATOM_BYTES;
    static constexpr int STAGES = BM <= 64 ? 8 : (BM <= 128 ? 6 : 4);
    static constexpr int TMEM_COLS = BM < 32 ? 32 : BM;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;     // + slack for 1024-byte alignment
};

// Atom `it` (64 columns; counted from the CTA's first chunk, 4 per chunk) -> ring stage and mbarrier phase.
// The two dequant warp sets take alternate chunks.  Each set owns one half of the ring and steps through it
// with its own atom counter, so every waiter (either set, the TMA lane, the MMA lane) comes back to a stage
// exactly one revolution later.  That is what keeps the 1-bit phase parity of mbarrier waits unambiguous: a
// set that shared one ring with the other would revisit a stage only every second revolution and its parity
// wait would be satisfied by a stale phase.
template <int STAGES>
LLM_DEVICE void ring_slot(int it, int& stage, int& phase) {
    constexpr int D = STAGES / 2;
    static_assert(STAGES % 2 == 0 && D >= 2, "each warp set needs at least two stages");
    const int set = (it >> 2) & 1;
    const int j = ((it >> 3) << 2) | (it & 3);      // atom index within the set's own sequence
    stage = set * D + j % D;
    phase = (j / D) & 1;
}

// Sink of the dequant warps: acquires ring stages atom by atom and publishes them to the MMA warp.
template <int STAGES>
struct RingSink {
    uint32_t smem_base;      // first stage
    int stage_bytes;
    uint32_t full_bar, empty_bar;    // arrays of 8-byte barriers
    int it0;                 // atom index of this chunk's first atom, counted from the CTA's first chunk
    int row, lane;
    volatile int* abort_flag;
    bool ok;
    LLM_DEVICE void begin(int a, int n) {
        for (int i = 0; i < n; ++i) {
            int stage, phase;
            ring_slot<STAGES>(it0 + a + i, stage, phase);
            if (ok) ok = mbar_wait_warp(empty_bar + stage * 8, phase ^ 1, abort_flag);
        }
    }
    LLM_DEVICE void emit(int kg, uint4 v) {
        int stage, phase;
        ring_slot<STAGES>(it0 + (kg >> 3), stage, phase);
        const uint32_t dst = smem_base + stage * stage_bytes + row * 128 + ((((kg & 7) ^ row) & 7) << 4);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
    LLM_DEVICE void end(int a, int n) {
        fence_proxy_async();
        __syncwarp();                          // every lane's stores are fenced before lane 0 publishes the stage
        for (int i = 0; i < n; ++i) {
            int stage, phase;
            ring_slot<STAGES>(it0 + a + i, stage, phase);
            mbar_arrive_if(full_bar + stage * 8, lane == 0);
        }
    }
};


// Copier CTA of the fused all-gather.  The `copy_ctas` copiers are the first CTAs of the grid and live for the whole
// gather: each walks the m-tiles in the order the GEMM CTAs will need them (own rows first) and stages its slice of every
// tile from the owners' row buffers (symmetric memory; peers over NVLink) into the local staging buffer, bumping the
// tile's counter after each slice.  They never wait on the GEMM CTAs, so they cannot be starved by them.
template <int BM>
LLM_DEVICE void ag_copier(const GemmTcParams& p, int slice, int m_tiles) {
    const AgFuse& ag = p.ag;
    const int tid = threadIdx.x;
    __shared__ int s_ok;
    // this rank's rows are complete (stream order): tell every peer once per launch
    if (slice == 0 && tid < ag.world) red_release_sys_add(ag.avail[tid] + ag.rank, 1u);
    const int rot = (ag.rank * ag.rows_per_rank) / BM;
    const int row_units = p.k >> 3;                             // 16-byte units per row
    const int stride = ag.copy_ctas * blockDim.x;
    unsigned seen = 1u << ag.rank;                              // sources whose rows are known to be published
    for (int i = 0; i < m_tiles; ++i) {
        const int tile_m = (rot + i) % m_tiles;
        const int r0 = tile_m * BM, r1 = min(r0 + BM, p.m);
        const int s_first = r0 / ag.rows_per_rank, s_last = (r1 - 1) / ag.rows_per_rank;
        unsigned need = 0;
        for (int s = s_first; s <= s_last; ++s) need |= 1u << s;
        if (need & ~seen) {
            if (tid == 0) {
                int ok = 1;
                for (int s = s_first; s <= s_last && ok; ++s) {
                    if (seen & (1u << s)) continue;
                    const unsigned* f = ag.avail[ag.rank] + s;
                    ok = 0;
                    for (unsigned it = 0; it < ag.spin_limit; ++it) {
                        if ((int)(ld_acquire_sys(f) - (ag.epoch + 1u)) >= 0) { ok = 1; break; }
                        if (it > 4096) __nanosleep(64);
                    }
                }
                if (!ok && p.status) atomicExch(p.status, (int)STATUS_TIMEOUT);
                s_ok = ok;
            }
            __syncthreads();
            if (s_ok) seen |= need;
        }
        if ((need & ~seen) == 0) {
            constexpr int INFLIGHT = 8;                         // 16-byte loads each thread keeps in flight
            const int total = (r1 - r0) * row_units;
            for (int u = slice * blockDim.x + tid; u < total; u += INFLIGHT * stride) {
                uint4 v[INFLIGHT];
#pragma unroll
                for (int j = 0; j < INFLIGHT; ++j) {
                    const int uu = u + j * stride;
                    if (uu < total) {
                        const int row = r0 + uu / row_units;
                        const int sr = row / ag.rows_per_rank;
                        const uint4* src = reinterpret_cast<const uint4*>(ag.src[sr] + (size_t)(row - sr * ag.rows_per_rank) * p.k) + uu % row_units;
                        asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w) : "l"(src) : "memory");
                    }
                }
#pragma unroll
                for (int j = 0; j < INFLIGHT; ++j) {
                    const int uu = u + j * stride;
                    if (uu < total) reinterpret_cast<uint4*>(ag.stage + (size_t)(r0 + uu / row_units) * p.k)[uu % row_units] = v[j];
                }
            }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) atomicAdd(ag.staged + tile_m, 1u);         // counted even after a timeout so that nobody waits twice
    }
}

template <int FMT, int BM>
__global__ void __launch_bounds__(320, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmTcParams p) {
    using C = Cfg<BM>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[C::STAGES];
    __shared__ __align__(8) uint64_t s_empty[C::STAGES];
    __shared__ __align__(8) uint64_t s_accum;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort[2];
    __shared__ int s_last;
    __shared__ uint32_t s_grid[FMT == FMT_IQ3_S ? 512 : 1];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned long long t_entry;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_entry));
    // fused all-gather: a linear grid whose first `copy_ctas` CTAs stage the activation rows (ag_copier) and whose other
    // CTAs take the output tiles n-fastest, with the m-tiles rotated so that the rows this rank owns come first
    int tile_n = blockIdx.x, tile_m = blockIdx.y, n_tiles_grid = gridDim.x;
    if (p.ag_on) {
        const int n_copy = p.ag.copy_ctas;
        const int m_tiles = (p.m + BM - 1) / BM;
        n_tiles_grid = (p.n + 127) / 128;
        if ((int)blockIdx.x < n_copy) {
            if (blockIdx.z == 0) ag_copier<BM>(p, blockIdx.x, m_tiles);
            return;
        }
        const int lin = blockIdx.x - n_copy;
        tile_n = lin % n_tiles_grid;
        tile_m = (lin / n_tiles_grid + (p.ag.rank * p.ag.rows_per_rank) / BM) % m_tiles;
    }
    // grouped mode: which group and which of its m-tiles this CTA has (surplus CTAs of the over-sized grid leave at once,
    // before any barrier or tensor-memory allocation)
    int row_lo = 0, row_hi = p.m;
    const uint8_t* w_base = p.w;
    if (p.groups > 0) {
        const int j = blockIdx.y;
        if (j >= __ldg(p.group_tile_off + p.groups)) return;
        int lo = 0, hi = p.groups;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (__ldg(p.group_tile_off + mid) <= j) lo = mid; else hi = mid;
        }
        tile_m = j - __ldg(p.group_tile_off + lo);
        row_lo = __ldg(p.group_row_off + lo);
        row_hi = __ldg(p.group_row_off + lo + 1);
        w_base += (long long)lo * p.w_group_stride;
    }
    const int k_blocks = p.k / 256;
    const int per = (k_blocks + gridDim.z - 1) / gridDim.z;
    const int kb0 = blockIdx.z * per, kb1 = min(k_blocks, kb0 + per);
    const int n_it = max(kb1 - kb0, 0) * 4;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full_bar = smem_u32(s_full), empty_bar = smem_u32(s_empty), accum_bar = smem_u32(&s_accum);

    if (tid == 0) {
        s_abort[0] = 0; s_abort[1] = 0;
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar + s * 8, 5); mbar_init(empty_bar + s * 8, 1); }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (FMT == FMT_IQ3_S) {
        for (int i = tid; i < 512; i += blockDim.x) s_grid[i] = g_iq3s_grid[i];
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem;
    volatile int* abort_flag = s_abort;
    const int cta_lin = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;

    const bool timing = p.debug && (p.flags & 0x100);
    auto ts = [&](int slot) {
        if (timing) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            reinterpret_cast<unsigned long long*>(p.debug)[(size_t)cta_lin * 8 + slot] = t;
        }
    };
    auto trace = [&](int slot, int value) {
        if (p.debug && !timing) {
            volatile int* d = p.debug + (size_t)cta_lin * 8;
            d[slot] = value;
            __threadfence_system();
        }
    };
    if (tid == 0) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        ts(1);
        if (timing) reinterpret_cast<unsigned long long*>(p.debug)[(size_t)cta_lin * 8 + 0] = t_entry;
        if (timing) reinterpret_cast<unsigned long long*>(p.debug)[(size_t)cta_lin * 8 + 7] = smid;
        trace(0, (int)smid + 1);
        trace(1, (int)tmem_base);
    }

    if (warp < 8) {
        // ------------------------------ dequant producers ------------------------------
        const int g = warp & 3, set = warp >> 2;
        const uint8_t* wtile = w_base + (size_t)tile_n * k_blocks * FmtTraits<FMT>::CHUNK;
        RingSink<C::STAGES> sink{smem_base, C::STAGE_BYTES, full_bar, empty_bar, 0, g * 32 + lane, lane, abort_flag, true};
        int kb = kb0 + set;
        typename DequantBlock<FMT>::Regs regs;
        if (kb < kb1) regs = DequantBlock<FMT>::load(wtile + (size_t)kb * FmtTraits<FMT>::CHUNK, g, lane);
        for (; kb < kb1; kb += 2) {
            typename DequantBlock<FMT>::Regs nxt = regs;
            if (kb + 2 < kb1) nxt = DequantBlock<FMT>::load(wtile + (size_t)(kb + 2) * FmtTraits<FMT>::CHUNK, g, lane);
            sink.it0 = (kb - kb0) * 4;
            if constexpr (FMT == FMT_IQ3_S) DequantBlock<FMT>::process(regs, sink, s_grid);
            else DequantBlock<FMT>::process(regs, sink);
            regs = nxt;
        }
    } else if (warp == 8) {
        // ------------------------------ TMA producer (activations) ------------------------------
        if (elect_one()) {
            bool ok = true;
            if (p.ag_on) {
                // wait (bounded) until the copier CTAs have staged this m-tile, then order their generic-proxy stores
                // before this lane's async-proxy (TMA) reads
                const unsigned target = (unsigned)p.ag.copy_ctas;
                const unsigned* f = p.ag.staged + tile_m;
                ok = false;
                abort_flag[1] = 1;                 // the rest of the pipeline is legitimately stalled meanwhile
                for (unsigned i = 0; i < p.ag.spin_limit; ++i) {
                    if ((int)(ld_acquire_gpu(f) - target) >= 0) { ok = true; break; }
                    if (i > 1024) __nanosleep(64);
                }
                abort_flag[1] = 0;
                if (!ok) abort_flag[0] = 1;
                asm volatile("fence.proxy.async;" ::: "memory");
            }
            for (int it = 0; it < n_it && ok; ++it) {
                int stage, phase;
                ring_slot<C::STAGES>(it, stage, phase);
                ok = mbar_wait(empty_bar + stage * 8, phase ^ 1, abort_flag);
                if (!ok) break;
                mbar_arrive_expect_tx(full_bar + stage * 8, C::B_ATOM_BYTES);
                tma_load_2d(smem_base + stage * C::STAGE_BYTES + A_ATOM_BYTES, &tmap_x, kb0 * 256 + it * 64, row_lo + tile_m * BM,
                            full_bar + stage * 8);
                trace(3, it + 1);
            }
        }
    } else {
        // ------------------------------ MMA issuer ------------------------------
        if (elect_one()) {
            constexpr uint32_t idesc = instr_desc(BM);
            bool ok = true;
            for (int it = 0; it < n_it && ok; ++it) {
                int stage, phase;
                ring_slot<C::STAGES>(it, stage, phase);
                ok = mbar_wait(full_bar + stage * 8, phase, abort_flag);
                if (!ok) break;
                if (it == 0) ts(2);
                tc_fence_after();
                const uint32_t a_addr = smem_base + stage * C::STAGE_BYTES;
                const uint64_t adesc = smem_desc_sw128(a_addr), bdesc = smem_desc_sw128(a_addr + A_ATOM_BYTES);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                    // advance 16 columns = 32 bytes inside the swizzle atom: +2 in the (addr >> 4) field
                    mma_f16(tmem_base, adesc + 2 * k4, bdesc + 2 * k4, idesc, (it > 0 || k4 > 0) ? 1u : 0u);
                }
                mma_commit(empty_bar + stage * 8);
                trace(2, it + 1);
            }
            if (ok) mma_commit(accum_bar);
            ts(3);
            trace(2, ok ? 1000 + n_it : -1);
        }
    }

    // ------------------------------ epilogue (warps 0-7) ------------------------------
    bool live = warp < 8;
    if (live && n_it > 0) live = mbar_wait(accum_bar, 0, abort_flag);
    if (*abort_flag) live = false;
    live = __all_sync(0xffffffffu, live);          // warp-uniform: the epilogue exchanges values between lanes
    if (tid == 0) ts(4);
    tc_fence_after();
    const int q = warp & 3, half = (warp >> 2) & 1;
    const int row_in_tile = q * 32 + lane;
    const int n_row = tile_n * 128 + row_in_tile;
    constexpr int HALF_COLS = BM / 2;
    constexpr int LOADS = HALF_COLS / 32;          // TMEM loads of 32 columns per warp
    static_assert(HALF_COLS % 32 == 0, "the epilogue reads the accumulator 32 columns at a time");
    const bool split = gridDim.z > 1;
    const uint32_t tmem_warp = tmem_base + ((uint32_t)(q * 32) << 16) + half * HALF_COLS;

    auto finish = [&](int c0, const float (&v)[32]) {
        // v[i]: value for token m0 + c0 + i, output row n_row
        const int m_base = row_lo + tile_m * BM + c0;
        if (p.epi == EPI_SWIGLU) {
            // rows of a 32-row group: 16 gate rows then the 16 matching up rows.  Lanes l and l + 16 hold one output
            // column; the lower lane finishes the even tokens and the upper lane the odd ones, so one exchange serves two.
            const int col = tile_n * 64 + q * 16 + (lane & 15);
            const bool lower = lane < 16;
            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)(m_base + (lower ? 0 : 1)) * p.out_stride + col;
            const bool col_ok = col < p.n / 2;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float got = __shfl_xor_sync(0xffffffffu, lower ? v[2 * j + 1] : v[2 * j], 16);
                const float gate = lower ? v[2 * j] : got, up = lower ? got : v[2 * j + 1];
                if (col_ok && m_base + 2 * j + (lower ? 0 : 1) < row_hi) o[(size_t)(2 * j) * p.out_stride] = __float2bfloat16(silu(gate) * up);
            }
            return;
        }
        if (n_row >= p.n) return;
        const float b = p.bias ? p.bias[n_row] : 0.f;
        if (p.epi == EPI_RESID) {
            float* h = static_cast<float*>(p.out) + (size_t)m_base * p.out_stride + n_row;
            float old[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) old[i] = (m_base + i < row_hi) ? h[(size_t)i * p.out_stride] : 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (m_base + i < row_hi) h[(size_t)i * p.out_stride] = old[i] + v[i] + b;
            return;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int m = m_base + i;
            if (m >= row_hi) continue;
            const size_t idx = (size_t)m * p.out_stride + n_row;
            if (p.out_f32) static_cast<float*>(p.out)[idx] = v[i] + b;
            else static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16(v[i] + b);
        }
    };
    // Walks this warp's accumulator columns 32 at a time, the next load in flight while `use` works on the current one.
    auto for_each_load = [&](auto&& use) {
        uint32_t ra[32], rb[32];
        tmem_ld32_issue(tmem_warp, ra);
#pragma unroll
        for (int c = 0; c < LOADS; c += 2) {
            tmem_wait_ld(ra);
            if (c + 1 < LOADS) tmem_ld32_issue(tmem_warp + (c + 1) * 32, rb);
            use(half * HALF_COLS + c * 32, ra);
            if (c + 1 < LOADS) {
                tmem_wait_ld(rb);
                if (c + 2 < LOADS) tmem_ld32_issue(tmem_warp + (c + 2) * 32, ra);
                use(half * HALF_COLS + (c + 1) * 32, rb);
            }
        }
    };

    if (p.rs_on) {
        // ---- fused reduce-scatter (RsFuse in gemm_tc.h): the partial tile goes to the owner of its rows ----
        // The operand ring is idle by now (every MMA has completed), so its first BM x 272 bytes serve as the transpose
        // buffer: each thread holds one output column for 32 tokens at a time, the wire wants 16-byte pieces of a row.
        constexpr int PITCH = 128 * 2 + 16;                   // bytes per token row of the tile (padded against bank conflicts)
        static_assert(BM * PITCH <= C::STAGES * C::STAGE_BYTES, "transpose buffer exceeds the operand ring");
        const RsFuse& rs = p.rs;
        if (warp < 8 && live) {
            auto stash = [&](int c0, const float (&v)[32]) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const uint32_t a = smem_base + (c0 + i) * PITCH + row_in_tile * 2;
                    const __nv_bfloat16 b = __float2bfloat16(v[i]);
                    asm volatile("st.shared.b16 [%0], %1;" ::"r"(a), "h"(*reinterpret_cast<const unsigned short*>(&b)) : "memory");
                }
            };
            if (n_it > 0) {
                for_each_load([&](int c0, const uint32_t (&r)[32]) {
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                    stash(c0, v);
                });
            } else {
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0.f;
                for (int c = 0; c < LOADS; ++c) stash(half * HALF_COLS + c * 32, v);
            }
        }
        if (warp < 8) asm volatile("bar.sync 1, 256;" ::: "memory");        // the eight epilogue warps only
        const int m0 = tile_m * BM;
        const int owner = m0 / rs.rows_per_rank;              // rows_per_rank is a multiple of BM: one owner per tile
        if (warp < 8 && live && owner < rs.world) {
            __nv_bfloat16* dst0 = rs.inbox[owner] + ((size_t)(rs.parity * rs.world + rs.rank) * rs.rows_per_rank + (m0 - owner * rs.rows_per_rank)) * rs.n_cap
                                  + (size_t)tile_n * 128;
            const int cols_ok = min(128, p.n - tile_n * 128);  // d_model is a multiple of 8
            for (int u = tid; u < BM * 16; u += 256) {
                const int t = u >> 4, c8 = (u & 15) * 8;
                if (m0 + t < p.m && c8 < cols_ok) {
                    uint4 v;
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_base + t * PITCH + c8 * 2));
                    *reinterpret_cast<uint4*>(dst0 + (size_t)t * rs.n_cap + c8) = v;
                }
            }
        }
        if (warp < 8) asm volatile("bar.sync 1, 256;" ::: "memory");        // every store of the tile precedes the one release below
        if (tid == 0 && live && owner < rs.world)
            red_release_sys_add(rs.flags[owner] + rs.parity * rs.flags_per_parity + (m0 - owner * rs.rows_per_rank) / BM, 1u);
    } else if (warp < 8 && !split && live) {
        if (n_it > 0) {
            for_each_load([&](int c0, const uint32_t (&r)[32]) {
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                finish(c0, v);
            });
        } else {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
            for (int c = 0; c < LOADS; ++c) finish(half * HALF_COLS + c * 32, v);
        }
    }
    if (split && !p.rs_on) {
        if (warp < 8 && live && n_it > 0) {
            for_each_load([&](int c0, const uint32_t (&r)[32]) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int m = tile_m * BM + c0 + i;
                    if (m < p.m) atomicAdd(&p.accum[(size_t)m * p.accum_stride + n_row], __uint_as_float(r[i]));
                }
            });
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned t = atomicAdd(&p.tickets[tile_m * n_tiles_grid + tile_n], 1u);
            s_last = (t == gridDim.z - 1);
            if (s_last) p.tickets[tile_m * n_tiles_grid + tile_n] = 0u;
        }
        __syncthreads();
        if (s_last && warp < 8) {
            __threadfence();
            for (int c = 0; c < LOADS; ++c) {
                const int c0 = half * HALF_COLS + c * 32;
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int m = tile_m * BM + c0 + i;
                    v[i] = 0.f;
                    if (m < p.m) {
                        float* a = &p.accum[(size_t)m * p.accum_stride + n_row];
                        v[i] = __ldcg(a);
                        __stcg(a, 0.f);
                    }
                }
                finish(c0, v);
            }
        }
    }

    // ------------------------------ teardown ------------------------------
    if (tid == 0) { trace(6, live ? 1 : -1); ts(5); }
    tc_fence_before();
    __syncthreads();
    if (tid == 0) ts(6);
    if (tid == 0) trace(6, *abort_flag ? -2 : 2);
    if (*abort_flag) {
        if (tid == 0 && p.status) atomicExch(p.status, (int)STATUS_TIMEOUT);
        // give copies that are still in flight time to land before this CTA's shared memory is handed on
        for (int i = 0; i < 2000; ++i) __nanosleep(100);
        __syncthreads();
    }
    if (warp == 9) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
        if (lane == 0) trace(7, 1);
    }
}

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

template <int FMT, int BM>
static cudaError_t launch_one(const GemmTcParams& p, int ksplit, cudaStream_t st) {
    using C = Cfg<BM>;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap tmap;
    const __nv_bfloat16* x_src = p.ag_on ? p.ag.stage : p.x;      // fused all-gather: the tensor map covers the local staging copy only
    const cuuint64_t dims[2] = {(cuuint64_t)p.k, (cuuint64_t)p.m};
    const cuuint64_t strides[1] = {(cuuint64_t)p.k * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)BM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(x_src), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<FMT, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    dim3 grid((p.n + 127) / 128, (p.m + BM - 1) / BM, ksplit);
    if (p.groups > 0) grid = dim3(grid.x, (p.m + BM - 1) / BM + p.groups, 1);     // at most one ragged tile per group more than m / BM
    if (p.ag_on) {                                   // per-m-tile counters of staged slices start from zero in every launch
        cudaError_t e = cudaMemsetAsync(p.ag.staged, 0, sizeof(unsigned) * grid.y, st);
        if (e != cudaSuccess) return e;
        grid = dim3(grid.x * grid.y + p.ag.copy_ctas, 1, ksplit);
    }
    gemm_tc_kernel<FMT, BM><<<grid, 320, C::SMEM_BYTES, st>>>(tmap, p);
    return cudaGetLastError();
}

}  // namespace tc

void gemm_tc_plan(int m, int n, int k, int ksplit_hint, int* block_m, int* ksplit) {
    const int bm = m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256));     // 32: persistent small-batch kernel
    const int tiles = ((n + 127) / 128) * ((m + bm - 1) / bm);
    const int kb = k / 256;
    int ks = ksplit_hint;
    if (ks <= 0) {
        // one CTA per SM: pick the split that minimises (waves of CTAs) x (chunks per CTA + fixed per-CTA cost)
        ks = 1;
        long best = -1;
        const int max_ks = kb < 16 ? kb : 16;
        for (int c = 1; c <= max_ks; ++c) {
            const long waves = ((long)tiles * c + 147) / 148;
            const long cost = waves * ((kb + c - 1) / c + (c > 1 ? 3 : 2));
            if (best < 0 || cost < best) { best = cost; ks = c; }
        }
    }
    if (ks > kb) ks = kb;
    if (ks < 1) ks = 1;
    *block_m = bm;
    *ksplit = ks;
}

int gemm_tc_rs_block_m(int m, int rows_per_rank) {
    int bm = m <= 64 ? 64 : (m <= 128 ? 128 : 256);
    while (rows_per_rank % bm) bm >>= 1;
    return bm;
}

template <int FMT>
static cudaError_t launch_fmt(const GemmTcParams& p, int bm, int ks, cudaStream_t st) {
    switch (bm) {
        case 64: return tc::launch_one<FMT, 64>(p, ks, st);
        case 128: return tc::launch_one<FMT, 128>(p, ks, st);
        case 256: return tc::launch_one<FMT, 256>(p, ks, st);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_gemm_tc(const GemmTcParams& p, cudaStream_t st) {
    if (p.m <= 0) return cudaSuccess;
    const void* xa = p.ag_on ? static_cast<const void*>(p.ag.stage) : static_cast<const void*>(p.x);
    if (p.k % 256 || (reinterpret_cast<uintptr_t>(xa) & 15)) return cudaErrorInvalidValue;
    int bm, ks;
    gemm_tc_plan(p.m, p.n, p.k, p.ksplit, &bm, &ks);
    if (p.ag_on) {
        if (p.m <= 32) bm = 64;                    // the fused all-gather lives in the large-tile kernel
        if (p.ag.world < 1 || p.ag.world > 8 || p.ag.copy_ctas < 1 || p.ag.rows_per_rank < 1) return cudaErrorInvalidValue;
    }
    if (p.groups > 0) {
        if (p.ag_on || p.rs_on || !p.group_row_off || !p.group_tile_off || p.epi == EPI_RESID) return cudaErrorInvalidValue;
        bm = p.group_bm;
        if (bm != 64 && bm != 128 && bm != 256) return cudaErrorInvalidValue;
        ks = 1;
    }
    if (p.rs_on) {
        // one owner per tile: the tile height must divide the rows every rank owns; no split-K (partials leave the GPU)
        if (p.rs.world < 1 || p.rs.world > 8 || p.rs.rows_per_rank < 64 || p.rs.rows_per_rank % 64 || p.bias || p.n % 8) return cudaErrorInvalidValue;
        if (bm < 64) bm = 64;
        while (p.rs.rows_per_rank % bm) bm >>= 1;
        ks = 1;
    }
    if (ks > 1 && (!p.accum || !p.tickets)) ks = 1;
    if (bm == 32 && !p.rs_on && p.groups == 0) return launch_gemm_tc_small(p, bm, (p.accum && p.tickets && p.ksplit != 1) ? 0 : 1, st);
    switch (p.fmt) {
        case FMT_Q4_K: return launch_fmt<FMT_Q4_K>(p, bm, ks, st);
        case FMT_Q5_K: return launch_fmt<FMT_Q5_K>(p, bm, ks, st);
        case FMT_Q6_K: return launch_fmt<FMT_Q6_K>(p, bm, ks, st);
        case FMT_Q8_0: return launch_fmt<FMT_Q8_0>(p, bm, ks, st);
        case FMT_Q4_0: return launch_fmt<FMT_Q4_0>(p, bm, ks, st);
        case FMT_IQ3_S: return launch_fmt<FMT_IQ3_S>(p, bm, ks, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace llm
