// ref_shim.cpp -- exposes the reference's own native CPU cross-check through a C ABI.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit contains none of the
// reference's code: it textually includes the reference's
// native/tests/reference_forward.cpp from where the reference tree is mounted
// (REF_ROOT, given on the compiler command line by oracle/Makefile) and, being
// the same translation unit, can call the file-local functions defined there:
//   gemv()     native/tests/reference_forward.cpp:67-75  (row-parallel, fp32 sum)
//   rmsnorm()  native/tests/reference_forward.cpp:78-91  (hidden size fixed at 2048)
// plus mc::fp8_e4m3_to_f32 from native/kernels/sm120/kernels.h:131-148.
// The output (oracle/_ref/libref_native.so) is a build product, never committed.
#define main mc_reference_forward_main
#include "tests/reference_forward.cpp"
#undef main
#include "kernels/sm120/kernels.h"

extern "C" {

// y[rows] = bf16( W[rows,in] . x[in] ) through the reference's gemv().
void ref_native_gemv(const uint16_t* x, const uint16_t* w, uint32_t rows, uint32_t in,
                     uint16_t* y) {
    bf16v xv(x, x + in), yv;
    gemv(xv, w, rows, in, yv);
    for (uint32_t r = 0; r < rows; ++r) y[r] = yv[r];
}

// out[2048] = rmsnorm(x[2048], w[2048]) through the reference's rmsnorm().
void ref_native_rmsnorm2048(const uint16_t* x, const uint16_t* w, uint16_t* out) {
    bf16v xv(x, x + H), ov;
    rmsnorm(xv, w, ov);
    for (uint32_t i = 0; i < H; ++i) out[i] = ov[i];
}

float ref_native_e4m3_to_f32(uint8_t code) { return mc::fp8_e4m3_to_f32(code); }

uint32_t ref_native_threads() {
    const unsigned hw = std::thread::hardware_concurrency();
    return hw == 0 ? 8u : (hw > 16u ? 16u : hw);
}

}  // extern "C"
