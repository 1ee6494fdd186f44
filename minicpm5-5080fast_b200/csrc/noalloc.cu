// noalloc.cu -- a split-K bf16 GEMV whose scratch memory is part of the library image.
//
// Some callers of this library may not allocate device memory themselves: a step
// that is being replayed from a CUDA graph, an executor whose arenas are frozen
// after start-up (the reference aborts on any allocation in steady state,
// native/runtime/memory_arena.cpp:38-46), or a plugin host that hands out no
// allocator at all.  The regular split-K call needs a caller-provided fp32
// partial buffer; this variant keeps that buffer in a file-scope device array
// instead, so the call needs nothing but its inputs and outputs.
#include "rows_dispatch.cuh"

namespace mcl {

// Upper bound on split_s * N of one call: 128 Ki floats = 512 KiB.  Every GPU
// whose context loads this library carries the array until the process exits.
constexpr uint32_t kStaticPartialFloats = 128u * 1024u;
static __device__ __align__(256) float g_static_partial[kStaticPartialFloats];

// Ordered merge of the S partial sums of each output (no atomics).
__global__ void static_splitk_merge_kernel(const float* __restrict__ partial, uint32_t S, uint32_t N,
                                           uint16_t* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float acc = 0.f;
    for (uint32_t s = 0; s < S; ++s) acc += partial[(size_t)s * N + n];
    y[n] = f32_to_bf16_bits(acc);
}

// Device address of the array for the current device.  In host code the array's
// name is only a handle, so the address is asked for once per device (with that
// device current) and remembered.
static mc_status_t static_partial_ptr(float** out) {
    static float* cached[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("mc_sm100_decode_gemv_splitk_static: cannot identify the current device: %s",
                  cudaGetErrorString(e));
        return MC_E_CUDA;
    }
    if (cached[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_partial);
        if (e != cudaSuccess || p == nullptr) {
            set_error("mc_sm100_decode_gemv_splitk_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return MC_E_CUDA;
        }
        cached[dev] = p;
    }
    *out = cached[dev];
    return MC_OK;
}

}  // namespace mcl

using namespace mcl;

extern "C" mc_status_t mc_sm100_decode_gemv_splitk_static(const uint16_t* d_w, const uint16_t* d_x,
                                                          uint16_t* d_y, uint32_t N, uint32_t K,
                                                          uint32_t split_s, void* stream, int32_t pdl) {
    clear_error();
    if (d_w == nullptr || d_x == nullptr || d_y == nullptr || N == 0 || K == 0 || (K & 7u) != 0 ||
        !aligned16(d_w) || !aligned16(d_x) || split_s < 2u || K % split_s != 0u || (K / split_s) % 8u != 0u) {
        set_error("mc_sm100_decode_gemv_splitk_static: invalid args (N=%u K=%u S=%u)", N, K, split_s);
        return MC_E_INVALID_ARGUMENT;
    }
    if ((uint64_t)split_s * N > kStaticPartialFloats) {
        set_error("mc_sm100_decode_gemv_splitk_static: split_s*N = %llu exceeds the built-in scratch of %u floats; "
                  "use mc_sm100_decode_gemv with a caller-provided partial buffer",
                  (unsigned long long)split_s * N, kStaticPartialFloats);
        return MC_E_UNSUPPORTED;
    }
    float* partial = nullptr;
    const mc_status_t ps = static_partial_ptr(&partial);
    if (ps != MC_OK) return ps;
    const cudaStream_t st = (cudaStream_t)stream;
    RowsArgs a{};
    a.w = d_w; a.x = d_x; a.y = d_y; a.N = N; a.K = K; a.y_stride = N; a.kseg = K / split_s;
    a.partial = partial;
    // every (segment, row) slot that the merge reads is written by this launch:
    // nothing in the array has to start at zero.
    const mc_status_t s = launch_rows<2, MATH_MIXED>(1, PRO_NONE, EPI_PARTIAL, a, split_s, st, pdl != 0);
    if (s != MC_OK) return s;
    (void)launch(static_splitk_merge_kernel, dim3((N + 255u) / 256u), dim3(256), 0, st, pdl != 0,
                 (const float*)partial, split_s, N, d_y);
    MCL_CHECK_LAUNCH("static_splitk_merge");
    return MC_OK;
}
