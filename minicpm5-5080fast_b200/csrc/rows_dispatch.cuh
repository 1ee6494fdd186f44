// rows_dispatch.cuh -- picks an instantiation of gemv_rows_kernel for a call.
//
// The template space (weight type, math form, M, prologue, epilogue, tile
// shape) is compiled in four translation units (rows_inst_*.cu), one per
// (weight type, math form); this header holds the switch that maps run-time
// arguments onto them.
#pragma once

#include "gemv_rows.cuh"

namespace mcl {

// Tile shapes: SHORT keeps a whole row of K <= 2304 (bf16) / 2560 (e4m3) in
// flight per lane in one batch; LONG walks longer rows in batches.
struct RowsShape { int R, U, T, B; };

template <int WB> struct ShapeOf;
template <> struct ShapeOf<2> {
    static constexpr RowsShape kShort{2, 9, 512, 1};
    static constexpr RowsShape kLong{2, 8, 512, 1};
};
template <> struct ShapeOf<1> {
    static constexpr RowsShape kShort{2, 5, 512, 2};
    static constexpr RowsShape kLong{2, 6, 512, 2};
};

// resident CTAs per SM for a tile shape (what the launch bounds guarantee)
constexpr int ctas_per_sm(const RowsShape& s) { return s.B; }

template <int WB, int MATH, int M, int PRO, int EPI, int R, int U, int T, int B>
inline mc_status_t launch_rows_one(const RowsArgs& a, uint32_t splits, cudaStream_t stream, bool pdl) {
    auto kern = gemv_rows_kernel<WB, M, R, U, PRO, EPI, MATH, T, B>;
    const size_t smem = (size_t)M * a.kseg * 2u;
    if (smem > 200u * 1024u) {
        set_error("gemv rows: activation tile of %zu bytes does not fit in shared memory", smem);
        return MC_E_UNSUPPORTED;
    }
    static SmemOptIn optin;   // per instantiation
    const cudaError_t e = optin.ensure(kern, smem);
    if (e != cudaSuccess) {
        set_error("gemv rows: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        return MC_E_CUDA;
    }
    const uint32_t groups = (a.N + R - 1) / R;
    const uint32_t resident = (uint32_t)(sm_count() * B);
    uint32_t gx = groups < resident ? groups : resident;
    if (EPI == EPI_ARGMAX && gx > kArgmaxCands) gx = kArgmaxCands;  // bounded stage buffer
    RowsArgs b = a;     // a.pf arrives as the raw hint (ptr, bytes); cut it into one slice per CTA
    b.pf = make_prefetch_args(NextWeights{a.pf.ptr, a.pf.bytes}, gx * splits);
    (void)launch(kern, dim3(gx, splits), dim3(T), smem, stream, pdl, b);
    MCL_CHECK_LAUNCH("gemv_rows");
    return MC_OK;
}

template <int WB, int MATH, int M, int PRO, int EPI>
inline mc_status_t launch_rows_shape(const RowsArgs& a, uint32_t splits, cudaStream_t stream, bool pdl) {
    constexpr RowsShape S = ShapeOf<WB>::kShort, L = ShapeOf<WB>::kLong;
    const uint32_t per_lane = (a.kseg * WB / 16u + 31u) / 32u;
    if (per_lane <= (uint32_t)S.U)
        return launch_rows_one<WB, MATH, M, PRO, EPI, S.R, S.U, S.T, S.B>(a, splits, stream, pdl);
    return launch_rows_one<WB, MATH, M, PRO, EPI, L.R, L.U, L.T, L.B>(a, splits, stream, pdl);
}

// Entry of one translation unit.  M in [1,4]; supported (PRO, EPI) pairs:
// M == 1: PRO_NONE with every epilogue, PRO_RESNORM with STORE / SWIGLU / ARGMAX,
// PRO_SWIGLU with STORE;
// M  > 1: PRO_NONE with STORE / SWIGLU / ARGMAX.
template <int WB, int MATH>
mc_status_t launch_rows(int M, int pro, int epi, const RowsArgs& a, uint32_t splits,
                        cudaStream_t stream, bool pdl);

#define MCL_ROWS_CASE(MV, PV, EV) \
    if (M == MV && pro == PV && epi == EV) \
        return launch_rows_shape<WB, MATH, MV, PV, EV>(a, splits, stream, pdl);

#define MCL_DEFINE_LAUNCH_ROWS(WBV, MATHV)                                               \
    template <>                                                                          \
    mc_status_t launch_rows<WBV, MATHV>(int M, int pro, int epi, const RowsArgs& a,      \
                                        uint32_t splits, cudaStream_t stream, bool pdl) { \
        constexpr int WB = WBV, MATH = MATHV;                                            \
        MCL_ROWS_CASE(1, PRO_NONE, EPI_STORE)                                            \
        MCL_ROWS_CASE(1, PRO_NONE, EPI_SWIGLU)                                           \
        MCL_ROWS_CASE(1, PRO_NONE, EPI_ARGMAX)                                           \
        MCL_ROWS_CASE(1, PRO_NONE, EPI_PARTIAL)                                          \
        MCL_ROWS_CASE(1, PRO_RESNORM, EPI_STORE)                                         \
        MCL_ROWS_CASE(1, PRO_RESNORM, EPI_SWIGLU)                                        \
        MCL_ROWS_CASE(1, PRO_RESNORM, EPI_ARGMAX)                                        \
        MCL_ROWS_CASE(1, PRO_SWIGLU, EPI_STORE)                                          \
        MCL_ROWS_CASE(2, PRO_NONE, EPI_STORE)                                            \
        MCL_ROWS_CASE(2, PRO_NONE, EPI_SWIGLU)                                           \
        MCL_ROWS_CASE(2, PRO_NONE, EPI_ARGMAX)                                           \
        MCL_ROWS_CASE(3, PRO_NONE, EPI_STORE)                                            \
        MCL_ROWS_CASE(3, PRO_NONE, EPI_SWIGLU)                                           \
        MCL_ROWS_CASE(3, PRO_NONE, EPI_ARGMAX)                                           \
        MCL_ROWS_CASE(4, PRO_NONE, EPI_STORE)                                            \
        MCL_ROWS_CASE(4, PRO_NONE, EPI_SWIGLU)                                           \
        MCL_ROWS_CASE(4, PRO_NONE, EPI_ARGMAX)                                           \
        set_error("gemv rows: no kernel for M=%d prologue=%d epilogue=%d", M, pro, epi); \
        return MC_E_UNSUPPORTED;                                                         \
    }

}  // namespace mcl
