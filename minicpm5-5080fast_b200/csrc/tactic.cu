// tactic.cu -- choosing the M = 1 bf16 GEMV tactic of a shape by timing it on the device.
//
// Stands for select_decode_gemv_tactics / run_decode_gemv (native/runtime/gemv_tactic.cpp:91-258,
// gemv_tactic.h:42-90): at session creation the reference times its candidates per shape and fixes the
// winner for the session (so that eager and replayed steps run the same kernels).  The candidates here are
// the row kernel (whose tile shape the static table of fast_dispatch.cuh picks) and split-K with S in
// {8, 4, 2}; the library-GEMM candidate of the reference does not exist.  The static table was tuned on
// 148 SMs and the shapes of one model; this entry point is for other SM counts and other shapes.
#include <cstring>

#include "common.cuh"

using namespace mcl;

namespace {

constexpr uint32_t kSplitMaxS = 8;          // gemv_tactic.h:43
constexpr uint32_t kSplitMaxN = 4096;       // gemv_tactic.h:45: split-K only for small N

// median of `reps` single-call timings; the optional flush buffer is rewritten before every call so that the
// weights come from HBM (the reference times back-to-back calls on L2-resident weights, gemv_tactic.cpp:60-88)
mc_status_t time_tactic(const uint16_t* d_w, const uint16_t* d_x, uint16_t* d_y, uint32_t N, uint32_t K, int32_t tactic, uint32_t S,
                        float* d_partial, void* d_flush, size_t flush_bytes, cudaStream_t st, float* us) {
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) {
        if (e0) cudaEventDestroy(e0);
        set_error("select tactic: cannot create events");
        return MC_E_CUDA;
    }
    constexpr int warm = 2, reps = 7;
    float t[reps];
    mc_status_t rc = MC_OK;
    for (int i = 0; i < warm + reps && rc == MC_OK; ++i) {
        if (d_flush != nullptr && flush_bytes != 0) (void)cudaMemsetAsync(d_flush, i, flush_bytes, st);
        (void)cudaEventRecord(e0, st);
        rc = mc_sm100_decode_gemv(d_w, d_x, d_y, N, K, tactic, S, d_partial, (void*)st, 0);
        (void)cudaEventRecord(e1, st);
        if (rc != MC_OK) break;
        if (cudaEventSynchronize(e1) != cudaSuccess) { set_error("select tactic: synchronise failed"); rc = MC_E_CUDA; break; }
        float ms = 0.f;
        (void)cudaEventElapsedTime(&ms, e0, e1);
        if (i >= warm) t[i - warm] = ms * 1e3f;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc != MC_OK) return rc;
    for (int i = 1; i < reps; ++i)
        for (int j = i; j > 0 && t[j] < t[j - 1]; --j) { const float x = t[j]; t[j] = t[j - 1]; t[j - 1] = x; }
    *us = t[reps / 2];
    return MC_OK;
}

}  // namespace

extern "C" {

// The reference's rule (gemv_tactic.h:42-56) with the block target taken from the current device: shapes whose
// row kernel already gives two CTAs' worth of warps per SM are not split; smaller ones try S = 8, 4, 2.
uint32_t mc_sm100_gemv_pick_split_s(uint32_t N, uint32_t K) {
    if (N == 0 || K == 0 || N > kSplitMaxN) return 1u;
    const uint32_t target = 2u * (uint32_t)sm_count();
    const uint32_t blocks = (N + 7u) / 8u;
    if (blocks >= target) return 1u;
    for (uint32_t S = kSplitMaxS; S >= 2u; S >>= 1)
        if (K % S == 0u && (K / S) % 8u == 0u && blocks * S >= target) return S;
    return 1u;
}

size_t mc_sm100_gemv_partial_floats(uint32_t max_n) { return (size_t)kSplitMaxS * max_n; }

mc_status_t mc_sm100_select_decode_gemv_tactic(const uint16_t* d_w, uint32_t N, uint32_t K, const uint16_t* d_x, uint16_t* d_y,
                                               float* d_partial, size_t partial_floats, void* d_flush, size_t flush_bytes,
                                               void* stream, mc_sm100_gemv_tactic_t* out) {
    clear_error();
    if (out == nullptr || d_w == nullptr || d_x == nullptr || d_y == nullptr || N == 0 || K == 0 || (K & 7u) != 0) {
        set_error("mc_sm100_select_decode_gemv_tactic: invalid args (N=%u K=%u)", N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    std::memset(out, 0, sizeof(*out));
    out->struct_size = sizeof(*out);
    out->tactic = MC_GEMV_TACTIC_ROWS;
    out->split_s = 1;
    const cudaStream_t st = (cudaStream_t)stream;
    mc_status_t rc = time_tactic(d_w, d_x, d_y, N, K, MC_GEMV_TACTIC_ROWS, 0, nullptr, d_flush, flush_bytes, st, &out->us_rows);
    if (rc != MC_OK) return rc;
    float best = out->us_rows;
    if (d_partial != nullptr && N <= kSplitMaxN) {
        for (uint32_t S = kSplitMaxS; S >= 2u; S >>= 1) {
            if (K % S != 0u || (K / S) % 8u != 0u || (size_t)S * N > partial_floats) continue;
            float us = 0.f;
            rc = time_tactic(d_w, d_x, d_y, N, K, MC_GEMV_TACTIC_SPLITK, S, d_partial, d_flush, flush_bytes, st, &us);
            if (rc != MC_OK) return rc;
            if (out->us_splitk == 0.f || us < out->us_splitk) { out->us_splitk = us; out->best_split_s = S; }
            if (us < best * 0.97f) { best = us; out->tactic = MC_GEMV_TACTIC_SPLITK; out->split_s = S; }   // a split has to win clearly: its sum order differs
        }
    }
    return MC_OK;
}

mc_status_t mc_sm100_run_decode_gemv(const mc_sm100_gemv_tactic_t* t, const uint16_t* d_w, const uint16_t* d_x, uint16_t* d_y, uint32_t N,
                                     uint32_t K, float* d_partial, void* stream, int32_t pdl) {
    clear_error();
    if (t == nullptr || t->struct_size != sizeof(*t)) { set_error("mc_sm100_run_decode_gemv: no tactic"); return MC_E_INVALID_ARGUMENT; }
    return mc_sm100_decode_gemv(d_w, d_x, d_y, N, K, t->tactic, t->tactic == MC_GEMV_TACTIC_SPLITK ? t->split_s : 0u,
                                t->tactic == MC_GEMV_TACTIC_SPLITK ? d_partial : nullptr, stream, pdl);
}

}  // extern "C"
