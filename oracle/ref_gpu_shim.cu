// ref_gpu_shim.cu -- the reference's own GPU kernels for this path, and the cuBLASLt call its
// batched path makes, behind a small C ABI so that the benchmark can time them BESIDE the library.
//
// BENCHMARK / TEST INFRASTRUCTURE ONLY; never linked into the shipped library.  This translation
// unit contains none of the reference's code.  oracle/Makefile compiles it together with the
// reference's native/kernels/sm120/gemv.cu, gemv_fp8.cu and native/runtime/error.cpp from where the
// reference tree is mounted, unmodified, for sm_100a (the kernels are plain SIMT code and build for
// any architecture), into oracle/_ref/libref_gpu.so -- a build product, never committed.
//   ref_gpu_decode_gemv      -> launch_decode_gemv, tactic rows   (native/kernels/sm120/gemv.cu:382-431)
//   ref_gpu_gemv_fp8         -> launch_gemv_fp8                   (gemv_fp8.cu:694-721)
//   ref_gpu_gemv_fp8_rows_m  -> launch_gemv_fp8_rows_m, M in 2..8 (gemv_fp8.cu:726-788)
//   ref_cublaslt_gemm_bf16   -> what GemmEngine::gemm_bf16 asks of cuBLASLt, restated from
//                               native/runtime/gemm.cpp:67-128 and :316-380: C = A^T B with A = W [K,N]
//                               column-major view of the row-major weight, bf16 in, fp32 compute, bf16
//                               out, the first heuristic that fits the caller's workspace, one plan per
//                               (M, N, K) built on first use.
#include <cstdint>
#include <map>
#include <tuple>

#include <cublasLt.h>
#include <cuda_runtime.h>

#include "kernels/sm120/kernels.h"

namespace {
struct Plan {
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
    cublasLtMatmulAlgo_t algo{};
};
cublasLtHandle_t g_handle = nullptr;
std::map<std::tuple<uint32_t, uint32_t, uint32_t>, Plan> g_plans;
}  // namespace

extern "C" {

const char* ref_gpu_last_error(void) { return mc_last_error(); }

int ref_gpu_decode_gemv(const uint16_t* d_w, const uint16_t* d_x, uint16_t* d_y, uint32_t N, uint32_t K, void* stream, int pdl) {
    return (int)launch_decode_gemv(d_w, d_x, d_y, N, K, mc::kGemvTacticRows, 0, nullptr, (cudaStream_t)stream, pdl != 0);
}

int ref_gpu_gemv_fp8(const uint8_t* d_w, const float* d_scale, const uint16_t* d_x, uint16_t* d_y, uint32_t N, uint32_t K, void* stream,
                     int pdl) {
    return (int)launch_gemv_fp8(d_w, d_scale, d_x, d_y, N, K, (cudaStream_t)stream, pdl != 0);
}

int ref_gpu_gemv_fp8_rows_m(const uint8_t* d_w, const float* d_scale, const uint16_t* d_x, uint16_t* d_y, uint32_t M, uint32_t N,
                            uint32_t K, void* stream, int pdl) {
    return (int)launch_gemv_fp8_rows_m(d_w, d_scale, d_x, d_y, M, N, K, (cudaStream_t)stream, pdl != 0);
}

// 0 = ok.  d_a = weight [N,K] row-major, d_b = activation [M,K] row-major, d_c = [M,N] row-major.
int ref_cublaslt_gemm_bf16(void* stream, void* d_workspace, size_t ws_size, uint32_t M, uint32_t N, uint32_t K, const void* d_a,
                           const void* d_b, void* d_c) {
    if (g_handle == nullptr && cublasLtCreate(&g_handle) != CUBLAS_STATUS_SUCCESS) return 1;
    const auto key = std::make_tuple(M, N, K);
    auto it = g_plans.find(key);
    if (it == g_plans.end()) {
        Plan p;
        if (cublasLtMatmulDescCreate(&p.op, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) return 2;
        const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
        cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta));
        cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb));
        if (cublasLtMatrixLayoutCreate(&p.la, CUDA_R_16BF, K, N, K) != CUBLAS_STATUS_SUCCESS ||
            cublasLtMatrixLayoutCreate(&p.lb, CUDA_R_16BF, K, M, K) != CUBLAS_STATUS_SUCCESS ||
            cublasLtMatrixLayoutCreate(&p.lc, CUDA_R_16BF, N, M, N) != CUBLAS_STATUS_SUCCESS)
            return 3;
        cublasLtMatmulPreference_t pref = nullptr;
        cublasLtMatmulPreferenceCreate(&pref);
        cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws_size, sizeof(ws_size));
        cublasLtMatmulHeuristicResult_t heur[4];
        int returned = 0;
        const cublasStatus_t st = cublasLtMatmulAlgoGetHeuristic(g_handle, p.op, p.la, p.lb, p.lc, p.lc, pref, 4, heur, &returned);
        cublasLtMatmulPreferenceDestroy(pref);
        if (st != CUBLAS_STATUS_SUCCESS || returned == 0) return 4;
        p.algo = heur[0].algo;
        it = g_plans.emplace(key, p).first;
    }
    const Plan& p = it->second;
    const float alpha = 1.0f, beta = 0.0f;
    const cublasStatus_t st = cublasLtMatmul(g_handle, p.op, &alpha, d_a, p.la, d_b, p.lb, &beta, d_c, p.lc, d_c, p.lc, &p.algo,
                                             d_workspace, ws_size, (cudaStream_t)stream);
    return st == CUBLAS_STATUS_SUCCESS ? 0 : 5;
}

}  // extern "C"
