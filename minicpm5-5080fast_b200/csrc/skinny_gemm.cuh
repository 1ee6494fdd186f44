// skinny_gemm.cuh -- interface of the tcgen05/TMEM batched-decode GEMM (4 < M <= 64).
#pragma once

#include "common.cuh"

namespace mcl {

enum : int { SKINNY_W_BF16 = 0, SKINNY_W_E4M3 = 1, SKINNY_W8A8 = 2 };

// Whether the tensor-core kernel takes this weight shape (wb = bytes per weight
// element).  Shapes it does not take are served by the CUDA-core family.
bool skinny_shape_ok(uint32_t N, uint32_t K, int wb);

// Global workspace the kernel needs: none (split-K partials are reduced through
// distributed shared memory inside a thread-block cluster).
size_t skinny_workspace_bytes(uint32_t M, uint32_t N, uint32_t K);

// y[M,N] = bf16( (w_scale[n] * x_scale[m]) * sum_k W[n,k] * X[m,k] ).
// SKINNY_W_BF16: W bf16, X bf16.  SKINNY_W_E4M3: W e4m3 widened to bf16 on the
// way into shared memory, X bf16 (weight-only arithmetic).  SKINNY_W8A8: W and X
// e4m3, kind::f8f6f4 (x passed through the uint16_t pointer type unchanged).
// swiglu: W rows are interleaved (gate_j, up_j); y[M, N/2] = bf16(silu(bf16 g) * bf16 u).
// x_pitch: elements between consecutive rows of x (0 = K): lets a GEMM read a column block of a wider matrix.
// out (sharded batched steps): the result goes into every rank's gathered buffer as tagged words instead of y
// (N, and N / 2 behind the SwiGLU epilogue, must then be even).
mc_status_t skinny_gemm(int mode, const void* w, const float* w_scale, const uint16_t* x,
                        const float* x_scale, uint16_t* y, uint32_t M, uint32_t N, uint32_t K,
                        bool swiglu, cudaStream_t stream, bool pdl, uint32_t x_pitch = 0,
                        const PeerOut* out = nullptr);

// 1 when a bounded wait inside the tensor-core kernel ran out since the last query (clears it), -1 on a CUDA error.
int skinny_take_error();

}  // namespace mcl
