// In-kernel all-reduce of one output tile across tensor-parallel ranks over NVLink peer memory.
//
// Used by the epilogues of the row-parallel GEMV / GEMM (attention output and FFN down projections): the CTA
// that holds a finished partial tile pushes it into every rank's inbox with plain peer stores, bumps a per-tile
// flag on every rank (red.release.sys), waits -- bounded -- until all ranks' contributions for this call have
// arrived in its own inbox and then adds their sum to the local residual stream.  One kernel therefore does
// GEMM + all-reduce + residual add; the reference runs GEMM, ncclAllReduce and an add kernel as three stages
// (reference: src/v2/models/qwen/QwenGraphBase.cpp:2937-3014, src/v2/collective/LocalTPContext.cpp:726).
//
// Protocol per tile t (every rank runs the same sequence of fused calls, all with d_model / 128 tiles):
//   e = epoch[t] (local call counter), parity = e & 1
//   inbox[r][parity][my_rank][m][n]  <- my partial, for every rank r          (peer stores)
//   CTA barrier; flags[r][t] += 1 on every rank r                             (red.release.sys: cumulative release)
//   spin (bounded) until flags[me][t] >= (e + 1) * size                        (acquire, system scope)
//   h[m][n] += sum_src inbox[me][parity][src][m][n]  (src order fixed, so all ranks compute identical bits)
// A rank can run at most one call ahead of a peer (it needs the peer's tiles of call c to finish call c), so two
// inbox parities suffice and monotone flags are never satisfied early.  No TMA and no multicast is involved.
//
// Two-phase variant (small-batch GEMM, groups of 4 or 8 ranks, >= two_phase_min_rows rows): rank d owns the column slice
// [d * 128 / size, (d + 1) * 128 / size) of every tile.  Phase 1 pushes each rank's partial of slice d into rs_inbox[d] and
// bumps flags[d][t]; the owner waits for `size` arrivals, sums the slice in rank order, pushes the result into every
// rank's ag_inbox and bumps flags2[.][t]; everyone waits for `size` arrivals there and adds the complete tile to h.
#pragma once
#include "common.cuh"

namespace llm {

constexpr int TP_MAX_RANKS = 8;

struct TpFuse {
    float* inbox[TP_MAX_RANKS];        // per rank: [2][size][rows_cap][n_cap] floats (symmetric memory)
    unsigned* flags[TP_MAX_RANKS];     // per rank: [n_cap / 128] arrival counters (symmetric memory)
    unsigned* epoch;                   // local: [n_cap / 128] call counters
    int* status;                       // local: set to STATUS_TIMEOUT when a wait gives up
    int rank, size, rows_cap, n_cap;
    unsigned spin_limit;               // iterations of the bounded wait
    // Two-phase variant (reduce-scatter then all-gather) for wider groups and larger tiles: the one-shot exchange sends
    // every partial tile to every rank (size x the tile bytes per rank), the two-phase one 2 x (size - 1) / size of them.
    int two_phase_min_rows;            // use it when size >= 4, size divides 128 and the call has at least this many rows (0: never)
    float* rs_inbox[TP_MAX_RANKS];     // per rank: [2][size src][rows_cap][n_cap / size]  partial column slices this rank reduces
    float* ag_inbox[TP_MAX_RANKS];     // per rank: [2][rows_cap][n_cap]                   reduced tiles, all column slices
    unsigned* flags2[TP_MAX_RANKS];    // per rank: [n_cap / 128] arrival counters of the all-gather phase
    unsigned* epoch2;                  // local: [n_cap / 128] two-phase call counters
};

LLM_DEVICE unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
LLM_DEVICE void red_release_sys_add(unsigned* p, unsigned v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Step 1: push.  v[i] is this thread's partial for (row m_first + i * m_step ... caller-defined), column n.
// The caller passes a functor row_of(i) -> activation row index (or -1 to skip).
template <int NV, class RowOf>
LLM_DEVICE void tp_push(const TpFuse& tp, unsigned epoch_val, int n, const float (&v)[NV], RowOf row_of) {
    const int parity = epoch_val & 1;
    for (int r = 0; r < tp.size; ++r) {
        float* base = tp.inbox[r] + ((size_t)(parity * tp.size + tp.rank) * tp.rows_cap) * tp.n_cap + n;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int m = row_of(i);
            if (m >= 0) base[(size_t)m * tp.n_cap] = v[i];
        }
    }
    // no fence here: the caller's CTA-wide barrier orders these stores before the signalling thread's
    // red.release.sys, whose release is cumulative over everything that happened before the barrier
}

// Step 2 (one thread per peer, after every pushing thread passed a barrier): signal.
LLM_DEVICE void tp_signal(const TpFuse& tp, int tile, int peer) { red_release_sys_add(tp.flags[peer] + tile, 1u); }

// Step 3 (one thread): bounded wait for all ranks of this call.  Returns false on timeout.
LLM_DEVICE bool tp_wait(const TpFuse& tp, int tile, unsigned epoch_val) {
    const unsigned target = (epoch_val + 1u) * (unsigned)tp.size;
    const unsigned* f = tp.flags[tp.rank] + tile;
    // a wait of this rank has run out already: the counters of the ranks no longer agree until the host has resynchronised
    // them, so the remaining calls of the step give up at once instead of waiting out the limit one after the other
    if (tp.status && *reinterpret_cast<volatile int*>(tp.status) != 0) return false;
    for (unsigned i = 0; i < tp.spin_limit; ++i) {
        // wrap-safe comparison of monotone counters
        if ((int)(ld_acquire_sys(f) - target) >= 0) return true;
        if (i > 4096) __nanosleep(64);       // the peer is normally a few microseconds away: poll hard first
    }
    if (tp.status) {
        // status[1..3]: which tile gave up, the count it saw and the count it wanted (a host-side report names them)
        tp.status[1] = tile; tp.status[2] = (int)ld_acquire_sys(f); tp.status[3] = (int)target;
        atomicExch(tp.status, (int)STATUS_TIMEOUT);
    }
    return false;
}

// Step 4: reduce this thread's elements from the local inbox (L1 bypassed: peers wrote the data).
template <int NV, class RowOf>
LLM_DEVICE void tp_reduce(const TpFuse& tp, unsigned epoch_val, int n, float (&v)[NV], RowOf row_of) {
    const int parity = epoch_val & 1;
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = 0.f;
    for (int src = 0; src < tp.size; ++src) {
        const float* base = tp.inbox[tp.rank] + ((size_t)(parity * tp.size + src) * tp.rows_cap) * tp.n_cap + n;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int m = row_of(i);
            if (m >= 0) v[i] += __ldcg(base + (size_t)m * tp.n_cap);
        }
    }
}

}  // namespace llm
