// Small-batch (1 <= M <= 64 rows; the engine uses it for 5..64) variant of the tcgen05 dequant GEMM: the weight-streaming,
// memory-bound regime of batched decode.  out[M, N] = x[M, K] * dequant(W)[N, K]^T with weights in the MMA M dimension.
//
// Differences from the large-tile kernel in gemm_tc.cu:
//   * the packed weight chunks (128 rows x 256 columns, ~14-34 KB) are fetched by one producer warp with 16-byte cp.async
//     into a deep shared-memory ring (an even number of slots), so HBM latency is hidden by bytes in flight rather than by
//     warps waiting on global loads; weights are constants, so under programmatic dependent launch the producer fills the
//     ring before the wait on the previous kernel;
//   * 16 dequant warps cooperate on every chunk: warp (g, a) converts the 64-column atom `a` of row group `g`
//     (lane == row), reading the packed bytes with ld.shared and storing the bf16 values straight into tensor
//     memory (tcgen05.st), from where the MMA takes its A operand: no shared-memory round trip for the weights.
//     The converted chunk lives in one of N_SETS operand sets (3; 2 for the formats whose warps alternate);
//   * two MMA issuer warps each issue half of EVERY chunk (issuer w takes atoms 2w and 2w+1): tcgen05.mma costs ~180
//     clocks to issue whatever its shape, and issue from different warps overlaps;
//   * persistent CTAs (one per SM) walk a contiguous range of (tile, chunk) work ("stream-K"): every SM streams
//     the same number of bytes, barriers / TMEM are set up once, and two TMEM accumulators let the MMAs of the
//     next tile start while the previous tile's epilogue drains; the finisher of a split tile loads the parked partial
//     sums before it waits for its own accumulator;
//   * SwiGLU pairs gate and up rows inside one warp (16 + 16 rows), so the epilogue needs a shuffle only.
// Warp roles: 0-15 dequant + epilogue, 16 raw-chunk producer, 17 activation TMA producer, 18-19 MMA issuers
// (18 also owns the TMEM allocation).
// Every barrier is visited by each of its waiters on every revolution (set counts and slot counts are chosen for that), so
// the 1-bit mbarrier parities are exact.
#include <cuda.h>

#include "formats_smem.cuh"
#include "launch.h"
#include "gemm_tc.h"
#include "gemv.h"
#include "tc_common.cuh"
#include "tp_fuse.cuh"

namespace llm {
namespace tcs {
using namespace tc5;

constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int N_DQ_WARPS = 16;
constexpr int THREADS = (N_DQ_WARPS + 4) * 32;      // + raw producer, activation producer, two MMA issuers

// Bounded wait.  abort_flag[0]: some wait of this CTA gave up (everybody leaves).  abort_flag[1]: the epilogue is inside its
// own bounded wait for a tensor-parallel peer; the pipeline behind it is legitimately stalled, so the count is held
// meanwhile (the peer wait has its own limit and reports through the status word).
// The timeline stamps are compiled in only for a tracing build (-DLLM_TRACE=1): a branch the compiler cannot prove
// warp-uniform costs a reconvergence sequence even when it is never taken, and the hot loops are sensitive to that.
#ifndef LLM_TRACE
#define LLM_TRACE 0
#endif
LLM_DEVICE void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}


template <int FMT, int BM> struct Cfg {
    static_assert(BM == 32, "the small-batch kernel is built for one 32-token tile");
    static constexpr int B_ATOM_BYTES = BM * 128;         // activation tile: BM tokens x 64 columns, 128B-swizzled
    // Formats converted by two alternating sets of eight warps (see TWO_SETS below): each warp set owns one operand set and
    // the raw ring has an even number of slots, so that every waiter meets each of its barriers on EVERY revolution.  A
    // waiter that meets a barrier only every second revolution can be two phases ahead of it, and a 1-bit parity wait
    // then passes on a stale phase (with three operand sets, or five raw slots, the alternating warp sets did exactly
    // that: an "unspecified launch failure" of the Q8_0 kernel on a 10240 x 5120 matrix).
    static constexpr bool TWO_SETS = (FMT == FMT_Q8_0 || FMT == FMT_IQ3_S);
    static constexpr int N_SETS = TWO_SETS ? 2 : 3;       // chunks in flight between the dequant warps and the MMA issuers
    static constexpr int N_B_STAGES = 4 * N_SETS;         // per chunk four 64-column activation atoms
    static constexpr int RING_BYTES = N_B_STAGES * B_ATOM_BYTES;
    static constexpr int CHUNK = FmtTraits<FMT>::CHUNK;
    static constexpr int BUDGET = 218 * 1024 - RING_BYTES;
    static constexpr int RAW_SLOTS_ = BUDGET / CHUNK;
    static constexpr int RAW_SLOTS = (RAW_SLOTS_ > 8 ? 8 : RAW_SLOTS_) & ~1;
    static_assert(RAW_SLOTS >= 2, "not enough shared memory for the raw chunk ring");
    static constexpr int SMEM_BYTES = RING_BYTES + RAW_SLOTS * CHUNK + 1024;
    static constexpr int COLS_PER_WARP = BM / 4;          // epilogue: 4 column parts x 4 lane quarters
    // Tensor memory map (512 columns x 128 lanes, all of it):
    //   [0, 128)    accumulators.  Control overhead per barrier wait / tcgen05.commit (~0.1 us each) dwarfs a 128x32x16
    //               MMA, so the pipeline synchronises per 256-column chunk (16 MMAs) and two issuer warps take alternate
    //               chunks, each into its own accumulator; the epilogue adds them up; the pair is double-buffered so the
    //               MMAs of unit i + 1 overlap the epilogue of unit i.
    //   [128, 512)  the dequantised weight operand (MMA "A from TMEM"): three chunks of 128 rows x 256 bf16 = 128 columns
    //               each.  Lane == weight row == dequant lane, so the dequant warps store their registers straight into
    //               TMEM (tcgen05.st) and the bf16 weights never pass through shared memory.  Issuing a chunk's 16 MMAs
    //               takes one lane ~0.85 us, longer than the ~0.6 us the 16 dequant warps need for a chunk; with only
    //               two operand slots the dequant warps waited for the slot of chunk c - 2 (period >= 0.8 us per
    //               chunk in a per-CTA timeline), a third slot takes that wait off the critical path.
    // Dequant warp organisation: formats whose conversion is light (Q8_0) or latency-heavy (IQ3_S grid lookups) run as two
    // sets of eight warps on alternate chunks (measured per-chunk period 1.59 -> 1.16 us and 2.20 -> 1.57 us); the
    // ALU-bound k-quants keep all sixteen warps on one chunk (two sets: 0.91 -> 1.10 us for Q4_K).
    static constexpr int DQ_WARPS_PER_CHUNK = TWO_SETS ? N_DQ_WARPS / 2 : N_DQ_WARPS;
    static constexpr int N_ISSUERS = 2;
    static constexpr int ACC_PER_ISSUER = 1;
    static constexpr int ACC_SET_COLS = N_ISSUERS * ACC_PER_ISSUER * BM;
    static constexpr int A_COLS_OFFSET = 2 * ACC_SET_COLS;
    static constexpr int A_CHUNK_COLS = 128;
    static constexpr int TMEM_COLS = 512;
    // Q4_K has a conversion with the atom index at run time (one copy of the code for the four warps of a scheduler)
    static constexpr bool RT_ATOM = (FMT == FMT_Q4_K);
    static_assert(A_COLS_OFFSET + N_SETS * A_CHUNK_COLS <= TMEM_COLS, "tensor memory map overflows");
};

// Sink that keeps a converted atom (64 bf16 of this lane's row, 32 packed pairs) in registers.
struct RegSink {
    uint32_t o[32];
    LLM_DEVICE void emit(int c, uint4 v) { o[4 * c] = v.x; o[4 * c + 1] = v.y; o[4 * c + 2] = v.z; o[4 * c + 3] = v.w; }
};

// Sink of a dequant warp: 8 bf16 (one uint4) -> 4 TMEM columns of this lane's row.
struct TmemSink {
    uint32_t taddr;         // lane quarter | first column of this atom in the current chunk's A region
    LLM_DEVICE void emit(int c, uint4 v) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr + c * 4), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
    // a whole 64-column atom of this lane's row (32 packed pairs) -> 32 TMEM columns, one instruction (measured alone, sixteen
    // warps: 940 bytes per clock and SM with .x32, 790 with .x8)
    LLM_DEVICE void emit64(const uint32_t (&r)[32]) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                     "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                     ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                     "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
                     "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
                     "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
    }
};

// Work distribution.  The (n_tile, chunk) pairs are flattened tile-major.  With scratch for partial sums
// (stream-K mode) CTA b takes the contiguous range [b*T/G, (b+1)*T/G) and therefore at most a few tiles, some
// of them partially; a partially covered tile is reduced through fp32 atomics and finished by the last
// contributor.  Without scratch every CTA takes whole tiles round-robin.
struct Unit { int tile, kb0, nkb, contributors; };
struct UnitIter {
    int k_blocks, n_tiles, total, G, b, streamk;
    int pos, end;
    LLM_DEVICE void init(int kb, int nt, int grid, int cta, int sk) {
        k_blocks = kb; n_tiles = nt; total = kb * nt; G = grid; b = cta; streamk = sk;
        if (streamk) { pos = (int)(((unsigned)b * (unsigned)total) / (unsigned)G); end = (int)(((unsigned)(b + 1) * (unsigned)total) / (unsigned)G); }
        else { pos = b; end = n_tiles; }
    }
    // 32-bit arithmetic: the launcher refuses problems with (chunks + 1) * grid >= 2^32 (64-bit division costs ~100 instructions)
    LLM_DEVICE int cta_of(int x) const { return (int)(((unsigned)(x + 1) * (unsigned)G - 1u) / (unsigned)total); }
    LLM_DEVICE bool next(Unit& u) {
        if (pos >= end) return false;
        if (streamk) {
            u.tile = pos / k_blocks;
            u.kb0 = pos - u.tile * k_blocks;
            u.nkb = min(k_blocks - u.kb0, end - pos);
            u.contributors = cta_of(u.tile * k_blocks + k_blocks - 1) - cta_of(u.tile * k_blocks) + 1;
            pos += u.nkb;
        } else {
            u.tile = pos; u.kb0 = 0; u.nkb = k_blocks; u.contributors = 1;
            pos += G;
        }
        return true;
    }
};

template <int FMT, int BM>
__global__ void __launch_bounds__(THREADS, 1) gemm_tc_small_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmTcParams p) {
    using C = Cfg<FMT, BM>;
    constexpr int R = C::RAW_SLOTS;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[C::N_SETS], s_empty[C::N_SETS], s_raw_full[R], s_raw_empty[R], s_acc_full[2], s_acc_empty[2], s_epi, s_sig, s_tick;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort[2], s_last, s_tp_ok;
    __shared__ unsigned s_tp_epoch, s_tp_epoch2;
    __shared__ uint32_t s_grid[FMT == FMT_IQ3_S ? 512 : 1];

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k_blocks = p.k / 256, n_tiles = (p.n + 127) / 128;
    const int streamk = p.flags & 2;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t raw_base = smem_base + C::RING_BYTES;       // activation ring first, raw weight chunks behind it
    const uint32_t full_bar = smem_u32(s_full), empty_bar = smem_u32(s_empty);
    const uint32_t rawf_bar = smem_u32(s_raw_full), rawe_bar = smem_u32(s_raw_empty);
    const uint32_t accf_bar = smem_u32(s_acc_full), acce_bar = smem_u32(s_acc_empty), epi_bar = smem_u32(&s_epi), sig_bar = smem_u32(&s_sig), tick_bar = smem_u32(&s_tick);

    if (tid == 0) {
        s_abort[0] = 0; s_abort[1] = 0;
        for (int s = 0; s < C::N_SETS; ++s) { mbar_init(full_bar + s * 8, C::DQ_WARPS_PER_CHUNK + 1); mbar_init(empty_bar + s * 8, C::N_ISSUERS); }
        for (int s = 0; s < R; ++s) { mbar_init(rawf_bar + s * 8, 1); mbar_init(rawe_bar + s * 8, C::DQ_WARPS_PER_CHUNK); }
        for (int s = 0; s < 2; ++s) { mbar_init(accf_bar + s * 8, C::N_ISSUERS); mbar_init(acce_bar + s * 8, N_DQ_WARPS); }
        mbar_init(epi_bar, N_DQ_WARPS);
        mbar_init(tick_bar, N_DQ_WARPS);
        mbar_init(sig_bar, N_DQ_WARPS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (FMT == FMT_IQ3_S) {
        for (int i = tid; i < 512; i += blockDim.x) s_grid[i] = g_iq3s_grid[i];
    }
    if (warp == N_DQ_WARPS + 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Everything above touched only this CTA's shared and tensor memory.  The weights are constants, so the raw-chunk producer
    // starts filling its ring at once (under programmatic dependent launch that overlaps the tail of the previous kernel) and
    // joins the wait only before its first wait on a ring slot; every other role waits here, before it reads activations or
    // writes outputs and scratch.
    if (warp != N_DQ_WARPS) pdl_wait();
    const uint32_t tmem_base = s_tmem;
    volatile int* abort_flag = s_abort;
    // optional timeline trace of CTA (flags >> 8): p.debug[role * 1024 + slot] = low 32 bits of the ns timer
    auto stamp = [&](int role, int slot) {
        if (LLM_TRACE && p.debug && (int)blockIdx.x == (p.flags >> 8) && slot < 1024) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            p.debug[role * 1024 + slot] = (int)(t & 0x7fffffff);
        }
    };
    // per-CTA start / end stamps: p.debug[4096 + 4 * cta + {0, 1, 2}] = start, end, end of dequant loop
    auto cta_stamp = [&](int slot) {
        if (LLM_TRACE && p.debug) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            p.debug[4096 + 4 * blockIdx.x + slot] = (int)(t & 0x7fffffff);
        }
    };
    if (tid == 0) cta_stamp(0);
    UnitIter it;
    it.init(k_blocks, n_tiles, gridDim.x, blockIdx.x, streamk);
    Unit u;

    // chunk counter cc -> half of the operand ring (stages set*4 .. set*4+3) and the phase of its barriers
    auto set_of = [](int cc) { return cc % C::N_SETS; };
    auto sphase_of = [](int cc) { return (cc / C::N_SETS) & 1; };

    if (warp < N_DQ_WARPS) {
        // ---------------- dequant + epilogue ----------------
        // TWO_SETS: two sets of eight warps take alternate chunks; warp (g, ah) of a set converts atoms 2 * ah and 2 * ah + 1
        // of row group g.  Otherwise all sixteen warps work on every chunk, warp (g, a) converting atom a.
        const int g = warp & 3, ws = C::TWO_SETS ? (warp >> 3) : 0, ah = (warp >> 2) & 1, a1 = warp >> 2;
        const int row = g * 32 + lane;
        const int q = g, part = warp >> 2;                 // epilogue: TMEM lane quarter q, column part `part`
        constexpr int CW = C::COLS_PER_WARP;
        TmemSink sink{0};
        int cc = 0, ui = 0, epi_syncs = 0, tick_syncs = 0;
        bool ok = true;
        // A chunk is published to the MMA issuers one step late (see the conversion loop): pend_* name the chunk that is owed.
        int pend_set = -1, pend_slot = -1;
        auto publish = [&]() {
            if (pend_set < 0) return;
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");      // warp-wide: every lane's stores are complete after it
            tc_fence_before();
            mbar_arrive_if(full_bar + pend_set * 8, lane == 0);       // this warp's part of the chunk's weight operand is in TMEM
            mbar_arrive_if(rawe_bar + pend_slot * 8, lane == 0);      // this warp no longer needs the raw chunk
            pend_set = -1;
        };
        // Epilogue of unit `ui_` (accumulator set ui_ & 1; its first chunk had counter cc0).  Returns false after a timeout.
        auto epilogue = [&](const Unit& u, int ui_, int cc0) -> bool {
            const int buf = ui_ & 1;
            if (warp == 0 && lane == 0) stamp(3, ui_ * 4 + 0);
            const int c0 = part * CW;
            // The finisher of a split tile (its first contributor) fetches the other contributors' parked partial sums BEFORE
            // it waits for its own accumulator: they were parked long ago (the others compute their share of the tile at the
            // start of their range), and both the counter round trip and the loads then run under the drain of this CTA's
            // last MMAs instead of after it.  A tile of k_blocks chunks spread over CTAs of >= 1 chunk has at most MAX_C
            // contributors in practice; more are handled one by one further down.
            constexpr int MAX_C = 4;
            float parked[MAX_C][CW];
            const bool use_slots = p.partials != nullptr;
            const int c_first = u.contributors > 1 ? it.cta_of(u.tile * k_blocks) : 0;
            const int c_last = u.contributors > 1 ? it.cta_of(u.tile * k_blocks + k_blocks - 1) : 0;
            const bool finisher = u.contributors > 1 && use_slots && (int)blockIdx.x == c_first;
            if (finisher) {
                const unsigned target = (unsigned)(N_DQ_WARPS * (u.contributors - 1));
                int got = 1;
                if (lane == 0) {
                    got = 0;
                    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
                        if (ld_acquire_gpu(&p.tickets[u.tile]) >= target) { got = 1; break; }
                        if (i > 64) { if (abort_flag[0]) break; __nanosleep(32); }
                    }
                    if (!got) abort_flag[0] = 1;
                }
                got = __shfl_sync(0xffffffffu, got, 0);
                __syncwarp();
                if (!got) return false;
                // Once every warp has seen the count, warp 0 puts the counter back for the next launch.  Only warp 0 waits, so
                // this rendezvous has a barrier of its own: on the barrier of the full rendezvous further down, the arrival of a
                // warp that is already one phase on would complete this phase before a slow warp has read the counter, and
                // that warp would then poll a counter that is back at zero until its limit (seen with tiles split between two
                // CTAs that finish together: four ranks, attention output projection).
                if (lane == 0) mbar_arrive(tick_bar);
                if (warp == 0) {
                    if (!mbar_wait(tick_bar, tick_syncs & 1, abort_flag)) return false;
                    if (lane == 0) p.tickets[u.tile] = 0u;
                }
                ++tick_syncs;
                const int nc = c_last - c_first + 1;
#pragma unroll
                for (int j = 1; j < MAX_C; ++j) {
                    const int c = c_first + j;
                    if (j < nc) {
                        const int c_pos = (int)(((unsigned)c * (unsigned)it.total) / (unsigned)it.G);
                        const float* theirs = p.partials + ((size_t)c * 2 + (c_pos / k_blocks == u.tile ? 0 : 1)) * (128 * BM);
#pragma unroll
                        for (int i = 0; i < CW; ++i) parked[j][i] = __ldcg(&theirs[(c0 + i) * 128 + row]);
                    }
                }
            }
            if (!mbar_wait(accf_bar + buf * 8, (ui_ >> 1) & 1, abort_flag)) return false;
            if (warp == 0 && lane == 0) stamp(3, ui_ * 4 + 1);
            tc_fence_after();
            float v[CW];
            // issuer w worked on this unit iff the unit has a chunk of parity w
            const bool has0 = true, has1 = true;      // both issuers work on every chunk (half of its K range each)
#pragma unroll
            for (int i = 0; i < CW; ++i) v[i] = 0.f;
#pragma unroll
            for (int acc = 0; acc < C::N_ISSUERS * C::ACC_PER_ISSUER; ++acc) {
                const bool valid = (acc < C::ACC_PER_ISSUER) ? has0 : has1;
                if (!valid) continue;
#pragma unroll
                for (int j = 0; j < CW / 8; ++j) {
                    uint32_t r[8];
                    tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + buf * C::ACC_SET_COLS + acc * BM + c0 + j * 8, r);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[j * 8 + i] += __uint_as_float(r[i]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar + buf * 8);   // accumulator may be overwritten by unit ui + 2
            const int n_row = u.tile * 128 + row;
            bool do_finish = true;
            if (u.contributors > 1) {
                // Split tile.  With a partials workspace every contributor parks its [32 tokens][128 rows] partial in its own
                // slot (slot 0: the CTA's first unit, slot 1: any later one -- a CTA has at most one split unit at each end
                // of its range) and the last arriver adds the slots up in CTA order; 4096 fp32 atomics per unit were
                // measured to cost several microseconds when all CTAs reach their unit boundary together.
                if (use_slots && !finisher) {
                    float* mine = p.partials + ((size_t)blockIdx.x * 2 + (ui_ > 0 ? 1 : 0)) * (128 * BM);
#pragma unroll
                    for (int i = 0; i < CW; ++i) __stcg(&mine[(c0 + i) * 128 + row], v[i]);
                } else if (!use_slots) {
#pragma unroll
                    for (int i = 0; i < CW; ++i) {
                        const int m = c0 + i;
                        if (m < p.m) atomicAdd(&p.accum[(size_t)m * p.accum_stride + n_row], v[i]);
                    }
                }
                if (use_slots) {
                    // The tile's first contributor finishes it: its part of the tile is the tail of its own chunk range and
                    // therefore the last to be computed (it has fetched the others' slots above).  The others hand their slot
                    // to the signal lane (in the activation producer's warp), which pays for the device-scope release (~2 us
                    // of waiting for the stores to be acknowledged) while these warps go back to converting weights.
                    __syncwarp();
                    if (!finisher) {
                        if (lane == 0) mbar_arrive(sig_bar);
                        do_finish = false;
                    }
                } else {
                __threadfence();
                __syncwarp();
                // all 16 epilogue warps meet (bounded) before and after the arrival ticket is taken
                if (lane == 0) mbar_arrive(epi_bar);
                ok = mbar_wait(epi_bar, epi_syncs & 1, abort_flag); ++epi_syncs;
                if (!ok) return false;
                if (tid == 0) {
                    const unsigned t = atomicAdd(&p.tickets[u.tile], 1u);
                    s_last = (t == (unsigned)u.contributors - 1);
                    if (s_last) p.tickets[u.tile] = 0u;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(epi_bar);
                ok = mbar_wait(epi_bar, epi_syncs & 1, abort_flag); ++epi_syncs;
                if (!ok) return false;
                do_finish = s_last != 0;
                }
                if (warp == 0 && lane == 0) stamp(3, ui_ * 4 + 2);
                if (do_finish) {
                    if (!use_slots) __threadfence();
                    if (use_slots) {
                        // contributors are the CTAs that own a chunk of this tile, in order; sum in that order (own registers
                        // first: the finisher is the first contributor) so that the result does not depend on who arrived last
                        const int nc = c_last - c_first + 1;
                        float sum[CW];
#pragma unroll
                        for (int i = 0; i < CW; ++i) sum[i] = v[i];
#pragma unroll
                        for (int j = 1; j < MAX_C; ++j) {
                            if (j >= nc) break;
#pragma unroll
                            for (int i = 0; i < CW; ++i) sum[i] += parked[j][i];
                        }
                        for (int c = c_first + MAX_C; c <= c_last; ++c) {        // more contributors than that: one by one
                            if (c == (int)blockIdx.x) {
#pragma unroll
                                for (int i = 0; i < CW; ++i) sum[i] += v[i];
                            } else {
                                const int c_pos = (int)(((unsigned)c * (unsigned)it.total) / (unsigned)it.G);
                                const float* theirs = p.partials + ((size_t)c * 2 + (c_pos / k_blocks == u.tile ? 0 : 1)) * (128 * BM);
#pragma unroll
                                for (int i = 0; i < CW; ++i) sum[i] += __ldcg(&theirs[(c0 + i) * 128 + row]);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < CW; ++i) v[i] = sum[i];
                    } else {
#pragma unroll
                        for (int i = 0; i < CW; ++i) {
                            const int m = c0 + i;
                            v[i] = 0.f;
                            if (m < p.m) {
                                float* acc = &p.accum[(size_t)m * p.accum_stride + n_row];
                                v[i] = __ldcg(acc);
                                __stcg(acc, 0.f);
                            }
                        }
                    }
                }
                // s_last is rewritten by the next split unit only after every warp passed the barrier above
            }
            if (do_finish) {
                if (p.epi == EPI_SWIGLU) {
                    // rows of a 32-row group: 16 gate rows then the 16 matching up rows -> pair lanes l and l + 16
                    const int col = u.tile * 64 + g * 16 + (lane & 15);
#pragma unroll
                    for (int i = 0; i < CW; ++i) {
                        const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
                        const int m = c0 + i;
                        if (lane < 16 && m < p.m && col < p.n / 2)
                            static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.out_stride + col] = __float2bfloat16(silu(v[i]) * other);
                    }
                } else if (p.tp != nullptr && p.epi == EPI_RESID) {
                    // fused tensor-parallel all-reduce of this tile, then the residual add (see tp_fuse.cuh);
                    // the 16 epilogue warps meet on the bounded mbarrier between the protocol steps
                    const TpFuse& tp = *p.tp;
                    auto epi_sync = [&]() {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(epi_bar);
                        const bool r = mbar_wait(epi_bar, epi_syncs & 1, abort_flag);
                        ++epi_syncs;
                        return r;
                    };
                    if (tid == 0) { s_tp_epoch = tp.epoch[u.tile]; s_tp_epoch2 = tp.epoch2[u.tile]; }
                    ok = epi_sync();
                    if (!ok) return false;
                    const unsigned e = s_tp_epoch;
                    auto row_of = [&](int i) { return (c0 + i) < p.m ? c0 + i : -1; };
                    if (tp.two_phase_min_rows > 0 && p.m >= tp.two_phase_min_rows) {
                        // ---- reduce-scatter + all-gather (see tp_fuse.cuh) ----
                        const int W = tp.size, slice = 128 / W, cols_rs = tp.n_cap / W;
                        const unsigned e2 = s_tp_epoch2;
                        const int par = e & 1, par2 = e2 & 1;
                        {   // phase 1: this thread's feature `row` belongs to the slice of rank `d`
                            const int d = row / slice, fo = row - d * slice;
                            float* dst = tp.rs_inbox[d] + ((size_t)(par * W + tp.rank) * tp.rows_cap) * cols_rs + u.tile * slice + fo;
                            const float b = (p.bias && tp.rank == 0 && n_row < p.n) ? p.bias[n_row] : 0.f;
#pragma unroll
                            for (int i = 0; i < CW; ++i) {
                                const int m = c0 + i;
                                if (m < p.m) dst[(size_t)m * cols_rs] = (n_row < p.n) ? v[i] + b : 0.f;
                            }
                        }
                        ok = epi_sync();
                        if (!ok) return false;
                        if (tid < W) tp_signal(tp, u.tile, tid);
                        if (tid == 0) {
                            abort_flag[1] = 1;
                            s_tp_ok = tp_wait(tp, u.tile, e) ? 1 : 0;
                            abort_flag[1] = 0;
                            tp.epoch[u.tile] = e + 1;
                        }
                        ok = epi_sync();
                        if (!ok) return false;
                        if (s_tp_ok) {
                            // phase 2a: reduce this rank's slice over all sources (fixed order) and hand it to every rank
                            const float* mine = tp.rs_inbox[tp.rank] + ((size_t)(par * W) * tp.rows_cap) * cols_rs + u.tile * slice;
                            for (int j = tid; j < p.m * slice; j += N_DQ_WARPS * 32) {
                                const int m = j / slice, fo = j - m * slice;
                                float r = 0.f;
                                for (int src = 0; src < W; ++src) r += __ldcg(mine + ((size_t)src * tp.rows_cap + m) * cols_rs + fo);
                                const size_t o = ((size_t)par2 * tp.rows_cap + m) * tp.n_cap + u.tile * 128 + tp.rank * slice + fo;
                                for (int dd = 0; dd < W; ++dd) tp.ag_inbox[dd][o] = r;
                            }
                        }
                        ok = epi_sync();
                        if (!ok) return false;
                        if (tid < W) red_release_sys_add(tp.flags2[tid] + u.tile, 1u);
                        if (tid == 0) {
                            abort_flag[1] = 1;
                            const unsigned target = (e2 + 1u) * (unsigned)W;
                            const unsigned* f2 = tp.flags2[tp.rank] + u.tile;
                            int got = 0;
                            const bool dead = tp.status && *reinterpret_cast<volatile int*>(tp.status) != 0;     // see tp_wait
                            for (unsigned it2 = 0; it2 < tp.spin_limit && !dead; ++it2) {
                                if ((int)(ld_acquire_sys(f2) - target) >= 0) { got = 1; break; }
                                if (it2 > 4096) __nanosleep(64);
                            }
                            if (!got && tp.status) {
                                tp.status[1] = u.tile | 0x10000; tp.status[2] = (int)ld_acquire_sys(f2); tp.status[3] = (int)target;
                                atomicExch(tp.status, (int)STATUS_TIMEOUT);
                            }
                            s_tp_ok = s_tp_ok && got;
                            abort_flag[1] = 0;
                            tp.epoch2[u.tile] = e2 + 1;
                        }
                        ok = epi_sync();
                        if (!ok) return false;
                        if (s_tp_ok && n_row < p.n) {
                            // phase 2b: the complete tile is in this rank's all-gather inbox
                            const float* full = tp.ag_inbox[tp.rank] + ((size_t)par2 * tp.rows_cap) * tp.n_cap + u.tile * 128 + row;
                            float* h = static_cast<float*>(p.out);
#pragma unroll
                            for (int i = 0; i < CW; ++i) {
                                const int m = c0 + i;
                                if (m < p.m) h[(size_t)m * p.out_stride + n_row] += __ldcg(full + (size_t)m * tp.n_cap);
                            }
                        }
                    } else {
                    if (n_row < p.n) {
                        if (p.bias && tp.rank == 0) {
#pragma unroll
                            for (int i = 0; i < CW; ++i) v[i] += p.bias[n_row];
                        }
                        tp_push<CW>(tp, e, n_row, v, row_of);
                    }
                    ok = epi_sync();
                    if (!ok) return false;
                    if (tid < tp.size) tp_signal(tp, u.tile, tid);
                    if (tid == 0) {
                        abort_flag[1] = 1;                     // hold the other warps' wait limits while the peer is awaited
                        s_tp_ok = tp_wait(tp, u.tile, e) ? 1 : 0;
                        abort_flag[1] = 0;
                        tp.epoch[u.tile] = e + 1;
                    }
                    ok = epi_sync();
                    if (!ok) return false;
                    if (s_tp_ok && n_row < p.n) {
                        tp_reduce<CW>(tp, e, n_row, v, row_of);
                        float* h = static_cast<float*>(p.out);
#pragma unroll
                        for (int i = 0; i < CW; ++i) {
                            const int m = c0 + i;
                            if (m < p.m) h[(size_t)m * p.out_stride + n_row] += v[i];
                        }
                    }
                    }
                } else if (n_row < p.n) {
                    const float b = p.bias ? p.bias[n_row] : 0.f;
                    if (p.epi == EPI_RESID) {
                        // residual add: all the loads first, then the stores (one L2 round trip instead of one per token)
                        float* h = static_cast<float*>(p.out) + n_row;
                        float hv[CW];
#pragma unroll
                        for (int i = 0; i < CW; ++i) hv[i] = (c0 + i < p.m) ? __ldcg(h + (size_t)(c0 + i) * p.out_stride) : 0.f;
#pragma unroll
                        for (int i = 0; i < CW; ++i)
                            if (c0 + i < p.m) h[(size_t)(c0 + i) * p.out_stride] = hv[i] + v[i] + b;
                    } else {
#pragma unroll
                        for (int i = 0; i < CW; ++i) {
                            const int m = c0 + i;
                            if (m >= p.m) continue;
                            const size_t idx = (size_t)m * p.out_stride + n_row;
                            const float o = v[i] + b;
                            if (p.out_f32) static_cast<float*>(p.out)[idx] = o;
                            else static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16(o);
                        }
                    }
                }
            }
            if (warp == 0 && lane == 0) stamp(3, ui_ * 4 + 3);
            return true;
        };
        // The epilogue of a unit is run two chunks into the next unit: by then its MMAs have completed, so the dequant warps
        // never sit out the drain of the operand ring, and the issuers work through those two chunks meanwhile.
        constexpr int DEFER = 2;
        Unit pu{};
        int p_ui = -1, p_cc0 = 0;
        auto flush = [&]() -> bool {
            if (p_ui < 0) return true;
            publish();
            const bool r = epilogue(pu, p_ui, p_cc0);
            p_ui = -1;
            return r;
        };
        // chunks [c_begin, c_end) of unit u
        auto convert = [&](int c_begin, int c_end) {
            for (int c = c_begin; c < c_end && ok; ++c, ++cc) {
                if (C::TWO_SETS && (cc & 1) != ws) continue;
                const int slot = cc % R, rphase = (cc / R) & 1;
                const int set = set_of(cc);
                ok = mbar_wait_warp(rawf_bar + slot * 8, rphase, abort_flag);
                if (LLM_TRACE && warp == 0 && lane == 0) stamp(0, cc * 4 + 0);
                // Q4_K: the packed bytes and the prepared scales go into registers now, so that the loads and the scale
                // arithmetic run under the wait for the operand slot instead of after it
                [[maybe_unused]] DequantAtomQ4KRt::Regs pre;
                if constexpr (C::RT_ATOM) {
                    if (ok) pre = DequantAtomQ4KRt::load(raw_base + slot * C::CHUNK, g, lane, a1);
                }
                if (ok) ok = mbar_wait_warp(empty_bar + set * 8, sphase_of(cc) ^ 1, abort_flag);
                if (LLM_TRACE && warp == 0 && lane == 0) stamp(0, cc * 4 + 1);
                if (!ok) return;
                const uint32_t raw = raw_base + slot * C::CHUNK;
                const uint32_t a_base = tmem_base + ((uint32_t)(g * 32) << 16) + C::A_COLS_OFFSET + set * C::A_CHUNK_COLS;
                if constexpr (C::TWO_SETS) {
                    if constexpr (FMT == FMT_IQ3_S) {
                        if (ah == 0) {
                            sink.taddr = a_base;      DequantAtom<FMT, 0>::run(raw, g, lane, sink, s_grid);
                            sink.taddr = a_base + 32; DequantAtom<FMT, 1>::run(raw, g, lane, sink, s_grid);
                        } else {
                            sink.taddr = a_base + 64; DequantAtom<FMT, 2>::run(raw, g, lane, sink, s_grid);
                            sink.taddr = a_base + 96; DequantAtom<FMT, 3>::run(raw, g, lane, sink, s_grid);
                        }
                    } else {
                        if (ah == 0) {
                            sink.taddr = a_base;      DequantAtom<FMT, 0>::run(raw, g, lane, sink);
                            sink.taddr = a_base + 32; DequantAtom<FMT, 1>::run(raw, g, lane, sink);
                        } else {
                            sink.taddr = a_base + 64; DequantAtom<FMT, 2>::run(raw, g, lane, sink);
                            sink.taddr = a_base + 96; DequantAtom<FMT, 3>::run(raw, g, lane, sink);
                        }
                    }
                } else {
                    // All sixteen warps on one chunk: the converted atom is built in registers, the PREVIOUS chunk is published
                    // (its tensor-memory stores have had this whole iteration to complete), and only then this chunk's single
                    // store is issued.  The MMA issue is cheap since it goes through elect.sync, and operand sets come free a
                    // chunk ahead of need, so the extra iteration of latency costs nothing.
                    RegSink rs;
                    if constexpr (C::RT_ATOM) {
                        DequantAtomQ4KRt::convert(pre, rs.o);
                    } else {
                        switch (a1) {
                            case 0: DequantAtom<FMT, 0>::run(raw, g, lane, rs); break;
                            case 1: DequantAtom<FMT, 1>::run(raw, g, lane, rs); break;
                            case 2: DequantAtom<FMT, 2>::run(raw, g, lane, rs); break;
                            default: DequantAtom<FMT, 3>::run(raw, g, lane, rs); break;
                        }
                    }
                    publish();
                    sink.taddr = a_base + a1 * 32;
                    sink.emit64(rs.o);
                    pend_set = set;
                    pend_slot = slot;
                }
                // The alternating warp sets publish at once: a set owns one operand set, so its next chunk's operand set frees
                // only after this chunk has been published and multiplied.
                if constexpr (C::TWO_SETS) {
                    pend_set = set;
                    pend_slot = slot;
                    publish();
                }
                if (LLM_TRACE && warp == 0 && lane == 0) stamp(0, cc * 4 + 2);
            }
        };
        while (ok && it.next(u)) {
            const int cc0 = cc;
            const int head = u.nkb < DEFER ? u.nkb : DEFER;
            convert(0, head);
            if (ok && p_ui >= 0) ok = flush();
            convert(head, u.nkb);
            if (!ok) break;
            pu = u; p_ui = ui; p_cc0 = cc0;                 // this unit's epilogue is owed
            ++ui;
        }
        if (ok) ok = flush();
    } else if (warp == N_DQ_WARPS) {
        // ---------------- raw chunk producer: one bulk copy per chunk ----------------
        // Measured on a ring of this shape with nothing behind it (148 CTAs, 18 KB chunks, 8 slots): one cp.async.bulk per
        // chunk streams 6.9 TB/s, a warp of 16-byte cp.async 4.0 TB/s (four such warps 6.7 TB/s), so the copy engine it is.
        if (elect_one()) {
            int cc = 0;
            bool ok = true;
            while (ok && it.next(u)) {
                const uint8_t* wsrc = p.w + ((size_t)u.tile * k_blocks + u.kb0) * C::CHUNK;
                for (int c = 0; c < u.nkb && ok; ++c, ++cc) {
                    const int slot = cc % R, rphase = (cc / R) & 1;
                    if (cc == R) pdl_wait();   // the first R slots start out empty: no wait, hence no time limit, before this
                    ok = mbar_wait(rawe_bar + slot * 8, rphase ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_arrive_expect_tx(rawf_bar + slot * 8, C::CHUNK);
                    bulk_load(raw_base + slot * C::CHUNK, wsrc + (size_t)c * C::CHUNK, C::CHUNK, rawf_bar + slot * 8);
                    stamp(1, cc);
                }
            }
        }
    } else if (warp == N_DQ_WARPS + 1) {
        // ---------------- activation tile producer (TMA): the four 64-column tiles of a chunk on one barrier ----------------
        if (lane == 16 && streamk && p.partials != nullptr) {
            // signal lane: once all dequant warps have parked their partial sums of a tile that another CTA finishes, one
            // release (cumulative over the mbarrier) publishes them to that CTA
            int n = 0;
            while (it.next(u)) {
                if (u.contributors > 1 && (int)blockIdx.x != it.cta_of(u.tile * k_blocks)) {
                    if (!mbar_wait(sig_bar, n & 1, abort_flag)) break;
                    red_release_gpu_add(&p.tickets[u.tile], (unsigned)N_DQ_WARPS);
                    ++n;
                }
            }
        }
        if (lane == 0) {
            int cc = 0;
            bool ok = true;
            while (ok && it.next(u)) {
                for (int c = 0; c < u.nkb && ok; ++c, ++cc) {
                    const int set = set_of(cc);
                    ok = mbar_wait(empty_bar + set * 8, sphase_of(cc) ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full_bar + set * 8, 4 * C::B_ATOM_BYTES);
#pragma unroll
                    for (int a = 0; a < 4; ++a)
                        tma_load_2d(smem_base + (set * 4 + a) * C::B_ATOM_BYTES, &tmap_x, (u.kb0 + c) * 256 + a * 64, 0,
                                    full_bar + set * 8);
                    stamp(6, cc);
                }
            }
        }
    } else {
        // ---------------- MMA issuers: warp w takes the chunks of parity w ----------------
        const int w = warp - (N_DQ_WARPS + 2);
        if (elect_one()) {
            constexpr uint32_t idesc = instr_desc(BM);
            int cc = 0, ui = 0;
            bool ok = true;
            while (ok && it.next(u)) {
                const int buf = ui & 1;
                ok = mbar_wait(acce_bar + buf * 8, ((ui >> 1) & 1) ^ 1, abort_flag);     // epilogue of unit ui - 2 has drained this accumulator set
                if (!ok) break;
                tc_fence_after();
                bool first = true;
                for (int c = 0; c < u.nkb && ok; ++c, ++cc) {
                    const int set = set_of(cc);
                    ok = mbar_wait(full_bar + set * 8, sphase_of(cc), abort_flag);
                    stamp(w == 0 ? 2 : 5, cc * 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t acc_base = tmem_base + buf * C::ACC_SET_COLS + w * C::ACC_PER_ISSUER * BM;
                    const uint32_t a_tmem = tmem_base + C::A_COLS_OFFSET + set * C::A_CHUNK_COLS;
#pragma unroll
                    for (int a2 = 0; a2 < 2; ++a2) {
                        const int a = 2 * w + a2;
                        const uint64_t bdesc = smem_desc_sw128(smem_base + (set * 4 + a) * C::B_ATOM_BYTES);
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)      // 16 columns of K = 8 TMEM columns of A, 32 bytes of the swizzled B row
                            mma_f16_ts(acc_base, a_tmem + a * 32 + k4 * 8, bdesc + 2 * k4, idesc, (first && a2 == 0 && k4 == 0) ? 0u : 1u);
                    }
                    mma_commit(empty_bar + set * 8);
                    stamp(w == 0 ? 2 : 5, cc * 2 + 1);
                    first = false;
                }
                if (ok) mma_commit(accf_bar + buf * 8);
                ++ui;
            }
        }
    }

    // ---------------- teardown ----------------
    if (tid == 0) { stamp(3, 1023); cta_stamp(2); }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0 && p.status) atomicExch(p.status, (int)STATUS_TIMEOUT);
        for (int i = 0; i < 2000; ++i) __nanosleep(100);   // let copies still in flight land before the CTA's memory is reused
        __syncthreads();
    }
    if (warp == N_DQ_WARPS + 2) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
    }
    if (tid == 0) cta_stamp(1);
}

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
    using C = Cfg<FMT, BM>;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    static_assert(C::CHUNK % 16 == 0 && C::RING_BYTES % 16 == 0, "bulk copies need 16-byte granularity");
    if (reinterpret_cast<uintptr_t>(p.w) & 15) return cudaErrorInvalidValue;      // the chunks arrive by bulk copy
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)p.k, (cuuint64_t)p.m};
    const cuuint64_t strides[1] = {(cuuint64_t)p.k * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)BM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(p.x), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_small_kernel<FMT, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    // persistent: one CTA per SM (or fewer when there is less work than that)
    GemmTcParams q = p;
    const int n_tiles = (p.n + 127) / 128, k_blocks = p.k / 256;
    if ((unsigned long long)(n_tiles * (long long)k_blocks + 1) * 148ull >= (1ull << 32)) return cudaErrorInvalidValue;   // 32-bit work indices
    const bool streamk = ksplit != 1 && p.accum && p.tickets;
    q.flags = (p.flags & ~2) | (streamk ? 2 : 0);
    const int units = streamk ? n_tiles * k_blocks : n_tiles;
    static int cached_sms = 0;
    if (!cached_sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&cached_sms, cudaDevAttrMultiProcessorCount, dev); }
    const int sms = cached_sms > 0 ? cached_sms : 148;
    int grid = units < sms ? units : sms;
    if (streamk) {
        // small problems: at least four chunks per CTA (the per-CTA start-up and epilogue cost a few chunks' worth of
        // time) and at most four contributors per tile (the finalizer fetches their partial sums in one round trip)
        const int g1 = (units + 3) / 4, g2 = 4 * n_tiles;
        int g = g1 < g2 ? g1 : g2;
        if (g < 1) g = 1;
        if (g < grid) grid = g;
    }
    if (grid > 148) q.partials = nullptr;            // the slot workspace is sized for 148 CTAs
    return launch_pdl(gemm_tc_small_kernel<FMT, BM>, dim3(grid), dim3(THREADS), C::SMEM_BYTES, st, tmap, q);
}

template <int FMT>
static cudaError_t launch_fmt(const GemmTcParams& p, int bm, int ks, cudaStream_t st) {
    if (bm == 32) return launch_one<FMT, 32>(p, ks, st);
    return cudaErrorInvalidValue;
}

}  // namespace tcs

cudaError_t launch_gemm_tc_small(const GemmTcParams& p, int bm, int ks, cudaStream_t st) {
    switch (p.fmt) {
        case FMT_Q4_K: return tcs::launch_fmt<FMT_Q4_K>(p, bm, ks, st);
        case FMT_Q5_K: return tcs::launch_fmt<FMT_Q5_K>(p, bm, ks, st);
        case FMT_Q6_K: return tcs::launch_fmt<FMT_Q6_K>(p, bm, ks, st);
        case FMT_Q8_0: return tcs::launch_fmt<FMT_Q8_0>(p, bm, ks, st);
        case FMT_Q4_0: return tcs::launch_fmt<FMT_Q4_0>(p, bm, ks, st);
        case FMT_IQ3_S: return tcs::launch_fmt<FMT_IQ3_S>(p, bm, ks, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace llm
