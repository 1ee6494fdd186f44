// gemm_mma_rows.cuh -- interface of the register-streaming batched GEMM for 2 <= M <= 16 (bf16 weights).
#pragma once

#include "common.cuh"

namespace mcl {

// How a weight of N rows is cut: blocks of `rows` rows, r of them per CTA at a time; worst_rows = rows the fullest SM
// walks through, balance = mean rows per SM / worst_rows (1 = perfectly even).
struct MmaRowsPlan { uint32_t rows, r, blocks, worst_rows; float balance; };
MmaRowsPlan mma_rows_plan(uint32_t N);                   // for the current device
MmaRowsPlan mma_rows_plan(uint32_t N, uint32_t sms);     // host logic alone

// Whether the kernel takes this call: bf16 weights, 2 <= M <= 16, K a multiple of 32, 16-byte aligned operands,
// an activation row pitch that is a multiple of 8 elements.
bool mma_rows_ok(uint32_t M, uint32_t N, uint32_t K, const void* w, const void* x, uint32_t x_pitch);

// y[M, N] = bf16( sum_k W[n, k] * X[m, k] ), W bf16 [N, K] row-major, X bf16 [M, x_pitch] (x_pitch = 0: K).
// swiglu: W rows are interleaved (gate_j, up_j); y[M, N / 2] = bf16(silu(bf16 g) * bf16 u).
// out (sharded batched steps): the result goes into every rank's gathered buffer as tagged words instead of y.
mc_status_t gemm_mma_rows(const void* w, const uint16_t* x, uint16_t* y, uint32_t M, uint32_t N, uint32_t K, bool swiglu,
                          cudaStream_t stream, bool pdl, uint32_t x_pitch = 0, const PeerOut* out = nullptr);

// The bf16 batched linear as the library dispatches it: this kernel up to the row count set with
// mma_rows_set_max_m (default 8, 0 = never) where a CTA owns a single row block, the tcgen05 kernel (skinny_gemm) otherwise.
mc_status_t batched_linear_bf16(const void* w, const uint16_t* x, uint16_t* y, uint32_t M, uint32_t N, uint32_t K, bool swiglu,
                                cudaStream_t stream, bool pdl, uint32_t x_pitch = 0, const PeerOut* out = nullptr);
void mma_rows_set_max_m(int max_m);

}  // namespace mcl
