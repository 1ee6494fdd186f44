// skinny_gemm.cu -- placeholder translation unit: the tensor-core kernel is not
// built yet, every shape reports "not taken" and goes to the CUDA-core family.
#include "skinny_gemm.cuh"

namespace mcl {

bool skinny_shape_ok(uint32_t, uint32_t, int) { return false; }
size_t skinny_workspace_bytes(uint32_t, uint32_t, uint32_t) { return 0; }

mc_status_t skinny_gemm(int, const void*, const float*, const uint16_t*, const float*, uint16_t*, uint32_t M,
                        uint32_t N, uint32_t K, void*, size_t, cudaStream_t, bool) {
    set_error("skinny_gemm: tensor-core path not built (M=%u N=%u K=%u)", M, N, K);
    return MC_E_UNSUPPORTED;
}

}  // namespace mcl
