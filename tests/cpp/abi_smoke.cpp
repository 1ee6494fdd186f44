// abi_smoke.cpp -- the library from a C++ host, through the reference's launcher names
// (include/mc_sm100a_launchers.hpp), with device memory from the CUDA runtime only.
// Mirrors the role of the reference's native/tests/abi_smoke.c: no Python, no torch.
// Exit code 0 = every check passed.  The expected values are computed here in double
// precision from the same bf16 / e4m3 inputs (products are exact, so only the final
// rounding differs): tolerance 2 bf16 ulp + 1e-3.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "mc_sm100a_launchers.hpp"

using namespace mc_sm100a;

static uint32_t g_state = 20260908u;
static float rnd() {   // uniform in (-1, 1)
    g_state = g_state * 1664525u + 1013904223u;
    return (float)((g_state >> 8) & 0xFFFFFF) / 8388608.0f - 1.0f;
}
static uint16_t to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static float from_bf16(uint16_t b) {
    const uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
static float from_e4m3(uint8_t c) {   // bit construction, 0x7F/0xFF = +-480 like the reference decoder
    const int e = (c >> 3) & 15, m = c & 7;
    const float v = e == 0 ? std::ldexp((float)m, -9) : std::ldexp(1.0f + (float)m / 8.0f, e - 7);
    return (c & 0x80) ? -v : v;
}
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); return 2; } } while (0)
#define MC(x) do { mc_status_t s_ = (x); if (s_ != MC_OK) { std::printf("mc_status %d at line %d: %s\n", (int)s_, __LINE__, mc_sm100_last_error()); return 3; } } while (0)

static int compare(const char* what, const std::vector<uint16_t>& got, const std::vector<double>& want) {
    int bad = 0;
    for (size_t i = 0; i < want.size(); ++i) {
        const double g = from_bf16(got[i]), tol = std::fabs(want[i]) * 2.0 / 128.0 + 1e-3;
        if (!(std::fabs(g - want[i]) <= tol)) { if (bad++ < 5) std::printf("%s[%zu]: got %g want %g\n", what, i, g, want[i]); }
    }
    std::printf("%s: %zu values, %d out of tolerance\n", what, want.size(), bad);
    return bad;
}

int main() {
    int32_t sms = 0, major = 0, minor = 0;
    uint64_t l2 = 0;
    MC(mc_sm100_device_check(&sms, &l2, &major, &minor));
    std::printf("device: cc %d.%d, %d SMs, L2 %llu MB\n", major, minor, sms, (unsigned long long)(l2 >> 20));
    const uint32_t N = 1000, K = 512;
    std::vector<uint16_t> w((size_t)N * K), x(K), y(N);
    std::vector<uint8_t> q((size_t)N * K);
    std::vector<float> sc(N);
    for (auto& v : w) v = to_bf16(0.02f * rnd());
    for (auto& v : x) v = to_bf16(rnd());
    for (auto& v : q) { g_state = g_state * 1664525u + 1013904223u; v = (uint8_t)(g_state >> 24); if ((v & 0x7F) == 0x7F) v &= 0xFE; }
    for (auto& v : sc) v = 0.001f * (1.0f + 0.5f * rnd());
    uint16_t *d_w, *d_x, *d_y;
    uint8_t* d_q;
    float* d_sc;
    CK(cudaMalloc(&d_w, w.size() * 2)); CK(cudaMalloc(&d_x, x.size() * 2)); CK(cudaMalloc(&d_y, y.size() * 2));
    CK(cudaMalloc(&d_q, q.size())); CK(cudaMalloc(&d_sc, sc.size() * 4));
    CK(cudaMemcpy(d_w, w.data(), w.size() * 2, cudaMemcpyHostToDevice)); CK(cudaMemcpy(d_x, x.data(), x.size() * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_q, q.data(), q.size(), cudaMemcpyHostToDevice)); CK(cudaMemcpy(d_sc, sc.data(), sc.size() * 4, cudaMemcpyHostToDevice));
    cudaStream_t st;
    CK(cudaStreamCreate(&st));
    int bad = 0;

    // bf16 GEMV, rows tactic, with and without programmatic dependent launch
    std::vector<double> want(N);
    for (uint32_t n = 0; n < N; ++n) { double s = 0; for (uint32_t k = 0; k < K; ++k) s += (double)from_bf16(w[(size_t)n * K + k]) * from_bf16(x[k]); want[n] = s; }
    for (int pdl = 0; pdl < 2; ++pdl) {
        CK(cudaMemsetAsync(d_y, 0xFF, y.size() * 2, st));
        MC(launch_decode_gemv(d_w, d_x, d_y, N, K, MC_GEMV_TACTIC_ROWS, 0, nullptr, st, pdl != 0));
        CK(cudaMemcpyAsync(y.data(), d_y, y.size() * 2, cudaMemcpyDeviceToHost, st)); CK(cudaStreamSynchronize(st));
        bad += compare(pdl ? "decode_gemv (pdl)" : "decode_gemv", y, want);
    }
    // e4m3 weight-only GEMV
    for (uint32_t n = 0; n < N; ++n) { double s = 0; for (uint32_t k = 0; k < K; ++k) s += (double)from_e4m3(q[(size_t)n * K + k]) * from_bf16(x[k]); want[n] = s * sc[n]; }
    CK(cudaMemsetAsync(d_y, 0xFF, y.size() * 2, st));
    MC(launch_gemv_fp8(d_q, d_sc, d_x, d_y, N, K, st));
    CK(cudaMemcpyAsync(y.data(), d_y, y.size() * 2, cudaMemcpyDeviceToHost, st)); CK(cudaStreamSynchronize(st));
    bad += compare("gemv_fp8", y, want);
    // batched bf16 GEMM through the engine-style call, M = 8 (tcgen05 path)
    {
        const uint32_t M = 8;
        std::vector<uint16_t> xm((size_t)M * K), ym((size_t)M * N);
        for (auto& v : xm) v = to_bf16(rnd());
        uint16_t *d_xm, *d_ym;
        CK(cudaMalloc(&d_xm, xm.size() * 2)); CK(cudaMalloc(&d_ym, ym.size() * 2));
        CK(cudaMemcpy(d_xm, xm.data(), xm.size() * 2, cudaMemcpyHostToDevice));
        GemmEngine eng;
        MC(eng.gemm_bf16(st, nullptr, 0, M, N, K, d_w, d_xm, d_ym));
        CK(cudaMemcpyAsync(ym.data(), d_ym, ym.size() * 2, cudaMemcpyDeviceToHost, st)); CK(cudaStreamSynchronize(st));
        std::vector<double> wm((size_t)M * N);
        for (uint32_t m = 0; m < M; ++m)
            for (uint32_t n = 0; n < N; ++n) { double s = 0; for (uint32_t k = 0; k < K; ++k) s += (double)from_bf16(w[(size_t)n * K + k]) * from_bf16(xm[(size_t)m * K + k]); wm[(size_t)m * N + n] = s; }
        bad += compare("gemm_bf16 M=8", ym, wm);
        cudaFree(d_xm); cudaFree(d_ym);
    }
    // error protocol: a bad argument comes back as a status and a message, nothing is launched
    if (launch_decode_gemv(nullptr, d_x, d_y, N, K, MC_GEMV_TACTIC_ROWS, 0, nullptr, st) != MC_E_INVALID_ARGUMENT || std::strlen(mc_sm100_last_error()) == 0) {
        std::printf("error protocol: expected MC_E_INVALID_ARGUMENT with a message\n");
        ++bad;
    }
    cudaFree(d_w); cudaFree(d_x); cudaFree(d_y); cudaFree(d_q); cudaFree(d_sc);
    std::printf(bad == 0 ? "ABI-SMOKE-OK\n" : "ABI-SMOKE-FAILED\n");
    return bad == 0 ? 0 : 1;
}
