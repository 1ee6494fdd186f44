// mc_sm100a_launchers.hpp -- the reference's internal launcher names on top of the C ABI.
//
// native/kernels/sm120/kernels.h declares the decode-path launchers as C++ functions taking a
// cudaStream_t and a trailing `bool pdl = false`.  An executor ported to B200 keeps its call
// sites and includes this header instead: every function below forwards, argument for argument,
// to the entry point of mc_sm100a_linear.h that replaces the launcher of the same name
// (kernels.h:666-672, 721-726, 735-748, 753-764, 774-779, 785-798; GemmEngine,
// native/runtime/gemm.h:33-110).  Status codes are the reference's mc_status_t values; the message
// of the last failure is mc_sm100_last_error().
#pragma once

#include <cuda_runtime.h>

#include "mc_sm100a_linear.h"

namespace mc_sm100a {

inline mc_status_t launch_decode_gemv(const uint16_t* d_w, const uint16_t* d_x, uint16_t* d_y, uint32_t N, uint32_t K, int tactic,
                                      uint32_t split_s, float* d_split_partial, cudaStream_t stream, bool pdl = false) {
    return mc_sm100_decode_gemv(d_w, d_x, d_y, N, K, tactic, split_s, d_split_partial, (void*)stream, pdl ? 1 : 0);
}
inline mc_status_t launch_gemv_fp8(const uint8_t* d_w, const float* d_scale, const uint16_t* d_x, uint16_t* d_y, uint32_t N,
                                   uint32_t K, cudaStream_t stream, bool pdl = false) {
    return mc_sm100_gemv_fp8(d_w, d_scale, d_x, d_y, N, K, (void*)stream, pdl ? 1 : 0);
}
inline mc_status_t launch_gemv_rows_prologue(const uint16_t* d_w, const uint16_t* d_res_in, const uint16_t* d_addend,
                                             const uint16_t* d_norm_w, uint16_t* d_res_out, uint16_t* d_y, uint32_t N, uint32_t n,
                                             float eps, cudaStream_t stream, bool pdl = false) {
    return mc_sm100_gemv_rows_prologue(d_w, d_res_in, d_addend, d_norm_w, d_res_out, d_y, N, n, eps, (void*)stream, pdl ? 1 : 0);
}
inline mc_status_t launch_gemv_fp8_prologue(const uint8_t* d_w, const float* d_scale, const uint16_t* d_res_in,
                                            const uint16_t* d_addend, const uint16_t* d_norm_w, uint16_t* d_res_out, uint16_t* d_y,
                                            uint32_t N, uint32_t n, float eps, cudaStream_t stream, bool pdl = false) {
    return mc_sm100_gemv_fp8_prologue(d_w, d_scale, d_res_in, d_addend, d_norm_w, d_res_out, d_y, N, n, eps, (void*)stream, pdl ? 1 : 0);
}
inline mc_status_t launch_gemv_rows_swiglu(const uint16_t* d_w, const uint16_t* d_gate_up, uint16_t* d_y, uint32_t N, uint32_t K,
                                           cudaStream_t stream, bool pdl = false) {
    return mc_sm100_gemv_rows_swiglu(d_w, d_gate_up, d_y, N, K, (void*)stream, pdl ? 1 : 0);
}
inline mc_status_t launch_gemv_fp8_swiglu(const uint8_t* d_w, const float* d_scale, const uint16_t* d_gate_up, uint16_t* d_y,
                                          uint32_t N, uint32_t K, cudaStream_t stream, bool pdl = false) {
    return mc_sm100_gemv_fp8_swiglu(d_w, d_scale, d_gate_up, d_y, N, K, (void*)stream, pdl ? 1 : 0);
}
inline mc_status_t launch_gemv_fp8_rows_m(const uint8_t* d_w, const float* d_scale, const uint16_t* d_x, uint16_t* d_y, uint32_t M,
                                          uint32_t N, uint32_t K, cudaStream_t stream, bool pdl = false) {
    return mc_sm100_gemv_fp8_rows_m(d_w, d_scale, d_x, d_y, M, N, K, (void*)stream, pdl ? 1 : 0);
}
inline mc_status_t launch_quant_rows(const uint16_t* d_x, uint8_t* d_xq, float* d_scale, uint32_t M, uint32_t K, cudaStream_t stream) {
    return mc_sm100_quant_rows(d_x, d_xq, d_scale, M, K, (void*)stream);
}
inline mc_status_t launch_post_scale_rows(uint16_t* d_y, const float* d_w_scale, const float* d_x_scale, uint32_t M, uint32_t N,
                                          cudaStream_t stream) {
    return mc_sm100_post_scale_rows(d_y, d_w_scale, d_x_scale, M, N, (void*)stream);
}

// GemmEngine (native/runtime/gemm.h:33-110) with the same member names and operand order (weight
// first).  The reference's engine owns a cuBLASLt handle and a plan cache; here there is no library
// handle and no plan to search, so init / destroy / prewarm_decode_shapes keep their place in the
// executor's start-up sequence (model.cpp, session.cpp) and have nothing to allocate: prewarm runs
// nothing because kernel selection is a pure function of (M, N, K) with no first-call search.
class GemmEngine {
public:
    GemmEngine() = default;
    GemmEngine(const GemmEngine&) = delete;
    GemmEngine& operator=(const GemmEngine&) = delete;

    mc_status_t init() { return mc_sm100_device_check(nullptr, nullptr, nullptr, nullptr); }
    void destroy() {}
    mc_status_t prewarm_decode_shapes(size_t /*ws_size*/) { return MC_OK; }

    mc_status_t gemm_bf16(cudaStream_t stream, void* d_workspace, size_t ws_size, uint32_t M, uint32_t N, uint32_t K, const void* d_w,
                          const void* d_x, void* d_y) const {
        return mc_sm100_gemm_bf16((void*)stream, d_workspace, ws_size, M, N, K, d_w, d_x, d_y);
    }
    // W8A8: activations quantised per row into the caller's scratch, then tcgen05 kind::f8f6f4 (gemm.h:64-90)
    mc_status_t gemm_fp8(cudaStream_t stream, void* d_workspace, size_t ws_size, uint32_t M, uint32_t N, uint32_t K,
                         const void* d_w_fp8, const float* d_w_scale, const uint16_t* d_x_bf16, uint16_t* d_y_bf16,
                         void* d_x_fp8_scratch, float* d_x_scale_scratch) const {
        return mc_sm100_gemm_fp8((void*)stream, d_workspace, ws_size, M, N, K, d_w_fp8, d_w_scale, d_x_bf16, d_y_bf16, d_x_fp8_scratch,
                                 d_x_scale_scratch);
    }
    mc_status_t gemm_fp8_q(cudaStream_t stream, void* d_workspace, size_t ws_size, uint32_t M, uint32_t N, uint32_t K,
                           const void* d_w_fp8, const float* d_w_scale, const void* d_x_fp8, const float* d_x_scale,
                           uint16_t* d_y_bf16) const {
        return mc_sm100_gemm_fp8_q((void*)stream, d_workspace, ws_size, M, N, K, d_w_fp8, d_w_scale, d_x_fp8, d_x_scale, d_y_bf16);
    }
    // 1 = both scale vectors applied inside the kernel (the reference's preferred OUTER_VEC mode, gemm.h:92-94);
    // the fall-back mode 2 (per-tensor scale + post-scale kernel) does not exist here.
    int fp8_scale_mode() const { return 1; }
    size_t cache_size() const { return 0; }
    static size_t workspace_bytes(uint32_t M, uint32_t N, uint32_t K) { return mc_sm100_gemm_workspace_bytes(M, N, K); }
};

}  // namespace mc_sm100a
