// fast_dispatch.cuh -- picks a tile shape of gemv_fast_kernel for an M = 1 call.
//
// The shape decides how much of the matrix is in flight before
// griddepcontrol.wait.  Small matrices get a shape whose warps cover every row
// in ONE round (all loads issued, and where registers allow also widened, before
// the wait); large matrices use the widest CTA and walk their rows in rounds.
#pragma once

#include "gemv_fast.cuh"

namespace mcl {

template <int WB, int R, int U, bool PRE, bool DB, int PRO, int EPI, int T, int MINB = 1>
inline mc_status_t launch_fast_one(const RowsArgs& a, cudaStream_t stream, bool pdl) {
    auto kern = gemv_fast_kernel<WB, R, U, PRE, DB, PRO, EPI, T, MINB>;
    const size_t smem = (size_t)a.K * (WB == 1 ? 4u : 2u) + (PRO == PRO_RESNORM ? (size_t)a.K * 4u : 0u);
    if (smem > 200u * 1024u) {
        set_error("gemv: activation of %zu bytes does not fit in shared memory", smem);
        return MC_E_UNSUPPORTED;
    }
    static SmemOptIn optin;
    const cudaError_t e = optin.ensure(kern, smem);
    if (e != cudaSuccess) {
        set_error("gemv: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        return MC_E_CUDA;
    }
    const uint32_t groups = (a.N + R - 1) / R;
    uint32_t gx = (uint32_t)sm_count();
    if (groups < gx) gx = groups;
    if (EPI == EPI_ARGMAX && gx > kArgmaxCands) gx = kArgmaxCands;
    RowsArgs b = a;     // a.pf arrives as the raw hint (ptr, bytes); cut it into one slice per CTA
    b.pf = make_prefetch_args(NextWeights{a.pf.ptr, a.pf.bytes}, gx);
    (void)launch(kern, dim3(gx), dim3(T), smem, stream, pdl, b);
    MCL_CHECK_LAUNCH("gemv_fast");
    return MC_OK;
}

// Tile shapes, from sweeps on B200 over the whole 40-layer chain (graph replay, PDL, every
// layer its own weights), one linear's shape varied at a time:
//  * a second register buffer (DB) and early widening (PRE) cost registers and were slower on
//    every shape, so neither is selected;
//  * e4m3: two rows per warp share each shared-memory read of x (lm_head 57 -> 45 us);
//  * the matrix that fits ONE round of a 512-thread CTA (o_proj) gains ~1 us per call from a
//    register budget of two CTAs per SM: the next kernel's CTA is then resident beside it and
//    streams its weights while this one computes.  Larger shapes lose more from the smaller
//    register file share than they gain.
template <int WB, int PRO, int EPI>
inline mc_status_t launch_fast_rows(const RowsArgs& a, cudaStream_t stream, bool pdl) {
    const uint32_t per_lane = (a.K * WB / 16u + 31u) / 32u;
    const uint32_t sms = (uint32_t)sm_count();
    if constexpr (WB == 2) {
        if (per_lane <= 9) {
            if (a.N <= 16u * sms) return launch_fast_one<2, 1, 9, false, false, PRO, EPI, 512, 2>(a, stream, pdl);   // one round, co-resident
            if (a.N <= 24u * sms) return launch_fast_one<2, 1, 9, false, false, PRO, EPI, 768>(a, stream, pdl);     // one round
            return launch_fast_one<2, 1, 9, false, false, PRO, EPI, 1024>(a, stream, pdl);
        }
        if (per_lane <= 24 && a.N <= 16u * sms) return launch_fast_one<2, 1, 24, false, false, PRO, EPI, 512>(a, stream, pdl);
        return launch_fast_one<2, 1, 12, false, false, PRO, EPI, 512>(a, stream, pdl);
    } else {
        if (per_lane <= 5) {
            if (a.N <= 32u * sms) return launch_fast_one<1, 2, 5, false, false, PRO, EPI, 512>(a, stream, pdl);     // one round of row pairs
            return launch_fast_one<1, 2, 5, false, false, PRO, EPI, 1024>(a, stream, pdl);
        }
        if (per_lane <= 12 && a.N <= 16u * sms) return launch_fast_one<1, 1, 12, false, false, PRO, EPI, 512>(a, stream, pdl);
        return launch_fast_one<1, 2, 6, false, false, PRO, EPI, 512>(a, stream, pdl);
    }
}

// SwiGLU epilogue over interleaved (gate, up) rows: a warp owns a pair
template <int WB, int PRO>
inline mc_status_t launch_fast_pairs(const RowsArgs& a, cudaStream_t stream, bool pdl) {
    const uint32_t per_lane = (a.K * WB / 16u + 31u) / 32u;
    if constexpr (WB == 2) {
        if (per_lane <= 9) {
            // A CTA walks its pairs in rounds of one pair per warp.  With 16 warps the last round of the
            // gate_up shape (38.9 pairs per CTA) is less than half full; spreading the pairs evenly over the
            // same number of rounds (13 - 14 warps) keeps every round's loads about equal: -0.55 us per call.
            const uint32_t sms = (uint32_t)sm_count();
            const uint32_t ppc = (a.N / 2u + sms - 1u) / sms, rounds = (ppc + 15u) / 16u;
            const uint32_t warps = rounds == 0u ? 16u : (ppc + rounds - 1u) / rounds + 1u;
            if (rounds > 1u && warps <= 12u) return launch_fast_one<2, 2, 9, false, false, PRO, EPI_SWIGLU, 384>(a, stream, pdl);
            if (rounds > 1u && warps <= 14u) return launch_fast_one<2, 2, 9, false, false, PRO, EPI_SWIGLU, 448>(a, stream, pdl);
            return launch_fast_one<2, 2, 9, false, false, PRO, EPI_SWIGLU, 512>(a, stream, pdl);
        }
        return launch_fast_one<2, 2, 12, false, false, PRO, EPI_SWIGLU, 512>(a, stream, pdl);
    } else {
        if (per_lane <= 5) {
            // same even-rounds rule with up to 24 warps: gate_up runs as two rounds of 20 warps
            const uint32_t sms = (uint32_t)sm_count();
            const uint32_t ppc = (a.N / 2u + sms - 1u) / sms, rounds = (ppc + 23u) / 24u;
            const uint32_t warps = rounds == 0u ? 24u : (ppc + rounds - 1u) / rounds;
            if (warps <= 20u) return launch_fast_one<1, 2, 5, false, false, PRO, EPI_SWIGLU, 640>(a, stream, pdl);
            return launch_fast_one<1, 2, 5, false, false, PRO, EPI_SWIGLU, 768>(a, stream, pdl);
        }
        return launch_fast_one<1, 2, 6, false, false, PRO, EPI_SWIGLU, 512>(a, stream, pdl);
    }
}

// Entry of one translation unit (fast_inst_w*.cu).
template <int WB>
mc_status_t launch_fast(int pro, int epi, const RowsArgs& a, cudaStream_t stream, bool pdl);

#define MCL_DEFINE_LAUNCH_FAST(WBV)                                                                  \
    template <>                                                                                      \
    mc_status_t launch_fast<WBV>(int pro, int epi, const RowsArgs& a, cudaStream_t stream, bool pdl) { \
        if (pro == PRO_NONE && epi == EPI_STORE) return launch_fast_rows<WBV, PRO_NONE, EPI_STORE>(a, stream, pdl);       \
        if (pro == PRO_NONE && epi == EPI_ARGMAX) return launch_fast_rows<WBV, PRO_NONE, EPI_ARGMAX>(a, stream, pdl);     \
        if (pro == PRO_NONE && epi == EPI_SWIGLU) return launch_fast_pairs<WBV, PRO_NONE>(a, stream, pdl);                \
        if (pro == PRO_RESNORM && epi == EPI_STORE) return launch_fast_rows<WBV, PRO_RESNORM, EPI_STORE>(a, stream, pdl); \
        if (pro == PRO_RESNORM && epi == EPI_ARGMAX) return launch_fast_rows<WBV, PRO_RESNORM, EPI_ARGMAX>(a, stream, pdl); \
        if (pro == PRO_RESNORM && epi == EPI_SWIGLU) return launch_fast_pairs<WBV, PRO_RESNORM>(a, stream, pdl);          \
        if (pro == PRO_SWIGLU && epi == EPI_STORE) return launch_fast_rows<WBV, PRO_SWIGLU, EPI_STORE>(a, stream, pdl);   \
        set_error("gemv: no kernel for prologue=%d epilogue=%d", pro, epi);                          \
        return MC_E_UNSUPPORTED;                                                                     \
    }

}  // namespace mcl
