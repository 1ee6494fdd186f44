// linear_api.cu -- the extern "C" boundary of the library: argument validation in
// the reference launchers' style, kernel selection, and the few helper kernels
// that are not part of the streaming GEMV family.
#include <atomic>
#include <thread>
#include <cstdarg>
#include <cstring>

#include "fast_dispatch.cuh"
#include "rows_dispatch.cuh"
#include "decode_chain.cuh"
#include "gemm_mma_rows.cuh"
#include "skinny_gemm.cuh"

namespace mcl {

// ---- diagnostics --------------------------------------------------------------------
static thread_local char g_err[512] = {0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
void clear_error() { g_err[0] = '\0'; }

// ---- L2 prefetch hint (thread-local, consumed by the next streaming launch) ----------------
static thread_local NextWeights g_next = {nullptr, 0};
NextWeights take_next_weights() {
    const NextWeights n = g_next;
    g_next = NextWeights{nullptr, 0};
    return n;
}
static thread_local int32_t* g_status_sink = nullptr;
void set_wait_status_sink(int32_t* d_status) { g_status_sink = d_status; }
int32_t* wait_status_sink() { return g_status_sink; }
// Defaults from measurements on B200.  The prefetch itself is OFF: with it the 40-layer bf16 M = 1 step
// went from 1.146 ms to 1.25 ms (bulk) / 1.28 ms (per line), because the lines a prefetch brings in
// are mostly gone when the next kernel asks for them (per-kernel counters, kernels serialised: L2 hit
// rate of the consumer's weight loads 1 - 3 % with or without the prefetch, while the step's DRAM reads grow
// from 106 to 172 MB per layer), and because an L2 hit streams at only ~1.5 x the HBM rate on this part
// (9.6 against 6.1 TB/s for the same reader).  Marking the demand loads evict-first is kept: -1.4 %.
static std::atomic<uint32_t> g_pf_mode{0}, g_pf_chunk{4096}, g_pf_evict_first{1};
static std::atomic<uint64_t> g_pf_cap{64ull << 20};
PrefetchConfig prefetch_config() {
    return PrefetchConfig{g_pf_mode.load(std::memory_order_relaxed), g_pf_chunk.load(std::memory_order_relaxed),
                          g_pf_evict_first.load(std::memory_order_relaxed), g_pf_cap.load(std::memory_order_relaxed)};
}

int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int v = cached[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

// Kernel form per weight type (index = bytes per weight element): 2 = the
// decode-chain kernel (gemv_fast_kernel, M = 1 only), 1 / 0 = gemv_rows_kernel with
// mixed-precision FMA / widen-then-FFMA.  All forms are compiled; the default is the
// measured winner and the debug hook lets a benchmark flip it.
constexpr int FORM_FAST = 2;
static std::atomic<int> g_math[3] = {{0}, {FORM_FAST}, {FORM_FAST}};

static mc_status_t rows(int wb, int M, int pro, int epi, const RowsArgs& a_in, uint32_t splits,
                        cudaStream_t st, bool pdl) {
    RowsArgs a = a_in;
    const NextWeights nw = take_next_weights();   // raw hint; the launcher cuts it into CTA slices
    a.pf.ptr = static_cast<const uint8_t*>(nw.ptr); a.pf.bytes = nw.bytes;
    int math = g_math[wb].load(std::memory_order_relaxed);
    if (math == FORM_FAST) {
        if (M == 1 && epi != EPI_PARTIAL && splits == 1)
            return wb == 2 ? launch_fast<2>(pro, epi, a, st, pdl) : launch_fast<1>(pro, epi, a, st, pdl);
        math = MATH_MIXED;
    }
    if (wb == 2)
        return math == MATH_MIXED ? launch_rows<2, MATH_MIXED>(M, pro, epi, a, splits, st, pdl)
                                  : launch_rows<2, MATH_CVT>(M, pro, epi, a, splits, st, pdl);
    return math == MATH_MIXED ? launch_rows<1, MATH_MIXED>(M, pro, epi, a, splits, st, pdl)
                              : launch_rows<1, MATH_CVT>(M, pro, epi, a, splits, st, pdl);
}

// ---- small kernels -------------------------------------------------------------------

// Fixed-order merge of split-K partials [S, M, N] -> bf16 y[M, N] (no atomics).
__global__ void splitk_merge_kernel(const float* __restrict__ partial, const float* __restrict__ scale,
                                    uint32_t S, uint32_t MN, uint32_t N, uint16_t* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= MN) return;
    float acc = 0.f;
    for (uint32_t s = 0; s < S; ++s) acc += partial[(size_t)s * MN + i];
    if (scale != nullptr) acc *= scale[i % N];
    y[i] = f32_to_bf16_bits(acc);
}

// Byte-wise e4m3 GEMV for shapes the vector path cannot take (K % 16 != 0 or
// misaligned pointers): one warp per output row, lanes stride K element-wise.
__global__ void gemv_fp8_bytes_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale,
                                      const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                                      uint32_t M, uint32_t N, uint32_t K) {
    pdl_trigger();
    pdl_wait();
    const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (row >= N) return;
    const uint8_t* wr = w + (size_t)row * K;
    for (uint32_t m = 0; m < M; ++m) {
        const uint16_t* xr = x + (size_t)m * K;
        float acc = 0.f;
        for (uint32_t k = lane; k < K; k += 32u)
            acc = fmaf(e4m3_to_f32(wr[k]), __uint_as_float((uint32_t)xr[k] << 16), acc);
        acc = warp_sum(acc);
        if (lane == 0) y[(size_t)m * N + row] = f32_to_bf16_bits(acc * scale[row]);
    }
}

// dst row 2j = src row j, dst row 2j+1 = src row I+j (16-byte or 4-byte granules).
__global__ void interleave_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                       uint32_t I, uint32_t row_bytes) {
    const uint32_t drow = blockIdx.x;  // 0 .. 2I-1
    const uint32_t srow = (drow & 1u) ? I + (drow >> 1) : (drow >> 1);
    const uint8_t* s = src + (size_t)srow * row_bytes;
    uint8_t* d = dst + (size_t)drow * row_bytes;
    if ((row_bytes & 15u) == 0u && (((uintptr_t)src | (uintptr_t)dst) & 15u) == 0u) {
        for (uint32_t i = threadIdx.x; i < row_bytes / 16u; i += blockDim.x)
            reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
    } else {
        for (uint32_t i = threadIdx.x; i < row_bytes; i += blockDim.x) d[i] = s[i];
    }
}

// ---- greedy argmax, two stages (semantics of native/kernels/sm120/sampling.cu:70-99) ----
constexpr uint32_t kArgmaxSlices = 64;   // stage-1 CTAs per logits row
constexpr uint32_t kArgmaxThreads = 512;

__device__ __forceinline__ void argmax_take(float& bv, int32_t& bi, float v, int32_t i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__device__ __forceinline__ void argmax_block_reduce(float& bv, int32_t& bi) {
    __shared__ float sv[32];
    __shared__ int32_t si[32];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, s);
        const int32_t oi = __shfl_xor_sync(0xffffffffu, bi, s);
        argmax_take(bv, bi, ov, oi);
    }
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const uint32_t nw = (blockDim.x + 31u) >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : INT32_MAX;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, s);
            const int32_t oi = __shfl_xor_sync(0xffffffffu, bi, s);
            argmax_take(bv, bi, ov, oi);
        }
    }
}

__global__ void argmax_stage1_kernel(const uint16_t* __restrict__ logits, uint32_t vocab,
                                     uint32_t row_stride, int32_t index_base,
                                     float* __restrict__ stage_val, int32_t* __restrict__ stage_idx) {
    pdl_trigger();
    pdl_wait();
    const uint32_t row = blockIdx.y, slice = blockIdx.x;
    const uint32_t per = (vocab + gridDim.x - 1) / gridDim.x;
    const uint32_t lo = slice * per, hi = min(vocab, lo + per);
    const uint16_t* lr = logits + (size_t)row * row_stride;
    float bv = -INFINITY;
    int32_t bi = INT32_MAX;
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x)
        argmax_take(bv, bi, __uint_as_float((uint32_t)lr[i] << 16), (int32_t)i + index_base);
    argmax_block_reduce(bv, bi);
    if (threadIdx.x == 0) {
        stage_val[(size_t)row * gridDim.x + slice] = bv;
        stage_idx[(size_t)row * gridDim.x + slice] = bi;
    }
}

// stage 2: reduce `cands` candidates per row laid out [row][cand] (row_major=1)
// or [cand][row] (row_major=0, the layout the fused lm_head epilogue writes).
__global__ void argmax_stage2_kernel(const float* __restrict__ stage_val,
                                     const int32_t* __restrict__ stage_idx, uint32_t cands,
                                     uint32_t n_rows, int row_major, int32_t* __restrict__ out_idx,
                                     float* __restrict__ out_val) {
    pdl_trigger();
    pdl_wait();
    const uint32_t row = blockIdx.x;
    float bv = -INFINITY;
    int32_t bi = INT32_MAX;
    for (uint32_t c = threadIdx.x; c < cands; c += blockDim.x) {
        const size_t at = row_major ? (size_t)row * cands + c : (size_t)c * n_rows + row;
        argmax_take(bv, bi, stage_val[at], stage_idx[at]);
    }
    argmax_block_reduce(bv, bi);
    if (threadIdx.x == 0) {
        out_idx[row] = bi;
        if (out_val != nullptr) out_val[row] = bv;
    }
}

// ---- activation quantiser of the W8A8 form (native/kernels/sm120/quant.cu:34-94) ----
__global__ void quant_rows_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ xq,
                                  float* __restrict__ scale, uint32_t M, uint32_t K) {
    __shared__ float wmax[8];
    __shared__ float s_row;
    const uint32_t t = threadIdx.x;
    for (uint32_t row = blockIdx.x; row < M; row += gridDim.x) {
        const uint16_t* xr = x + (size_t)row * K;
        float am = 0.f;
        for (uint32_t k = t; k < K; k += blockDim.x)
            am = fmaxf(am, fabsf(__uint_as_float((uint32_t)xr[k] << 16)));
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, s));
        if ((t & 31u) == 0u) wmax[t >> 5] = am;
        __syncthreads();
        if (t == 0) {
            float v = wmax[0];
            for (uint32_t w = 1; w < blockDim.x / 32u; ++w) v = fmaxf(v, wmax[w]);
            s_row = v;
            scale[row] = v > 0.f ? v / 448.f : 1.f;
        }
        __syncthreads();
        const float inv = s_row > 0.f ? 448.f / s_row : 0.f;
        uint8_t* qr = xq + (size_t)row * K;
        for (uint32_t k = t; k < K; k += blockDim.x) {
            const float v = __uint_as_float((uint32_t)xr[k] << 16) * inv;
            uint16_t packed;
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(0.0f), "f"(v));
            qr[k] = (uint8_t)(packed & 0xFFu);
        }
        __syncthreads();
    }
}

__global__ void post_scale_rows_kernel(uint16_t* __restrict__ y, const float* __restrict__ ws,
                                       const float* __restrict__ xs, uint32_t M, uint32_t N) {
    const size_t tot = (size_t)M * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < tot;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t m = (uint32_t)(i / N), n = (uint32_t)(i % N);
        float s = ws[n];
        if (xs != nullptr) s *= xs[m];
        y[i] = f32_to_bf16_bits(__uint_as_float((uint32_t)y[i] << 16) * s);
    }
}

// res[r,:] = bf16(res[r,:] + add[r,:]) in place (add may be null), then
// out[r,:] = bf16( res * rsqrt(mean(res^2) + eps) * w ) on the ROUNDED residual; one
// CTA per row (semantics of native/kernels/sm120/rmsnorm.cu:130-166).
__global__ void residual_rmsnorm_rows_kernel(uint16_t* __restrict__ res, const uint16_t* __restrict__ add,
                                             const uint16_t* __restrict__ w, uint16_t* __restrict__ out,
                                             uint32_t n, float eps, const TaggedIn tin, uint32_t* advance) {
    __shared__ float part[8];
    pdl_trigger();
    pdl_wait();
    if (tin.words != nullptr) {
        // the addend is a gathered buffer of tagged words (two elements each): poll, add, round -- a thread owns
        // the same pairs in the second pass below
        const uint32_t tag = (*tin.step - 1u) * tin.layers + tin.lsel;
        const uint64_t* tr = tin.words + (size_t)blockIdx.x * tin.pitch;
        uint16_t* rr2 = res + (size_t)blockIdx.x * n;
        uint16_t* orow2 = out + (size_t)blockIdx.x * n;
        float ss2 = 0.f;
        for (uint32_t i = threadIdx.x; i < n / 2u; i += blockDim.x) {
            const uint32_t ad = ld_tagged_pair(tr + i, tag, tin);
            const uint32_t rv = reinterpret_cast<const uint32_t*>(rr2)[i];
            const uint16_t r0 = f32_to_bf16_bits(__uint_as_float(rv << 16) + __uint_as_float(ad << 16));
            const uint16_t r1 = f32_to_bf16_bits(__uint_as_float(rv & 0xFFFF0000u) + __uint_as_float(ad & 0xFFFF0000u));
            reinterpret_cast<uint32_t*>(rr2)[i] = (uint32_t)r0 | ((uint32_t)r1 << 16);
            const float f0 = __uint_as_float((uint32_t)r0 << 16), f1 = __uint_as_float((uint32_t)r1 << 16);
            ss2 = fmaf(f0, f0, ss2);
            ss2 = fmaf(f1, f1, ss2);
        }
        ss2 = warp_sum(ss2);
        if ((threadIdx.x & 31u) == 0u) part[threadIdx.x >> 5] = ss2;
        __syncthreads();
        float tot2 = 0.f;
        for (uint32_t k = 0; k < blockDim.x / 32u; ++k) tot2 += part[k];
        const float inv2 = 1.0f / sqrtf(tot2 / (float)n + eps);
        for (uint32_t i = threadIdx.x; i < n / 2u; i += blockDim.x) {
            const uint32_t rv = reinterpret_cast<const uint32_t*>(rr2)[i], wv = reinterpret_cast<const uint32_t*>(w)[i];
            const uint16_t o0 = f32_to_bf16_bits(__uint_as_float(rv << 16) * inv2 * __uint_as_float(wv << 16));
            const uint16_t o1 = f32_to_bf16_bits(__uint_as_float(rv & 0xFFFF0000u) * inv2 * __uint_as_float(wv & 0xFFFF0000u));
            reinterpret_cast<uint32_t*>(orow2)[i] = (uint32_t)o0 | ((uint32_t)o1 << 16);
        }
        if (advance != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *advance = *advance + 1u;
        return;
    }
    uint16_t* rr = res + (size_t)blockIdx.x * n;
    const uint16_t* ar = add ? add + (size_t)blockIdx.x * n : nullptr;
    uint16_t* orow = out + (size_t)blockIdx.x * n;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float r = __uint_as_float((uint32_t)rr[i] << 16);
        if (ar != nullptr) {
            const uint16_t rb = f32_to_bf16_bits(r + __uint_as_float((uint32_t)ar[i] << 16));
            rr[i] = rb;
            r = __uint_as_float((uint32_t)rb << 16);
        }
        ss = fmaf(r, r, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31u) == 0u) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (uint32_t k = 0; k < blockDim.x / 32u; ++k) tot += part[k];
    const float inv = 1.0f / sqrtf(tot / (float)n + eps);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x)   // each thread re-reads only what it wrote
        orow[i] = f32_to_bf16_bits(__uint_as_float((uint32_t)rr[i] << 16) * inv * __uint_as_float((uint32_t)w[i] << 16));
    if (advance != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *advance = *advance + 1u;
}

// The same operation for widths that are a multiple of 8 and at most 8192: a thread owns one 16-byte chunk of the row and
// keeps it in registers, so the row is read once, the norm weights are in flight before the grid dependency resolves,
// and one barrier separates the loads from the stores.  Element arithmetic as above; only the order of the sum of
// squares differs.
__global__ void __launch_bounds__(1024) residual_rmsnorm_rows_vec_kernel(uint16_t* __restrict__ res, const uint16_t* __restrict__ add,
                                                                         const uint16_t* __restrict__ w, uint16_t* __restrict__ out,
                                                                         uint32_t n, float eps, const TaggedIn tin, uint32_t* advance) {
    __shared__ float part[32];
    const uint32_t c = threadIdx.x;
    const bool on = c < n / 8u;
    uint4 wv = make_uint4(0u, 0u, 0u, 0u);
    if (on) wv = __ldg(reinterpret_cast<const uint4*>(w) + c);
    pdl_trigger();
    pdl_wait();
    uint4* rrow = reinterpret_cast<uint4*>(res + (size_t)blockIdx.x * n);
    uint32_t r[4] = {0u, 0u, 0u, 0u}, a[4] = {0u, 0u, 0u, 0u};
    const bool tagged = tin.words != nullptr, adds = tagged || add != nullptr;
    if (on) {
        const uint4 rv = rrow[c];
        r[0] = rv.x; r[1] = rv.y; r[2] = rv.z; r[3] = rv.w;
        if (tagged) {
            const uint32_t tag = (*tin.step - 1u) * tin.layers + tin.lsel;
            const uint64_t* tr = tin.words + (size_t)blockIdx.x * tin.pitch + (size_t)c * 4u;
#pragma unroll
            for (int j = 0; j < 4; ++j) a[j] = ld_tagged_pair(tr + j, tag, tin);
        } else if (add != nullptr) {
            const uint4 av = reinterpret_cast<const uint4*>(add + (size_t)blockIdx.x * n)[c];
            a[0] = av.x; a[1] = av.y; a[2] = av.z; a[3] = av.w;
        }
    }
    float f[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float lo = __uint_as_float(r[j] << 16), hi = __uint_as_float(r[j] & 0xFFFF0000u);
        if (adds) {
            const uint16_t b0 = f32_to_bf16_bits(lo + __uint_as_float(a[j] << 16));
            const uint16_t b1 = f32_to_bf16_bits(hi + __uint_as_float(a[j] & 0xFFFF0000u));
            r[j] = (uint32_t)b0 | ((uint32_t)b1 << 16);
            lo = __uint_as_float((uint32_t)b0 << 16);
            hi = __uint_as_float((uint32_t)b1 << 16);
        }
        f[2 * j] = lo;
        f[2 * j + 1] = hi;
        ss = fmaf(lo, lo, ss);
        ss = fmaf(hi, hi, ss);
    }
    if (on && adds) rrow[c] = make_uint4(r[0], r[1], r[2], r[3]);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31u) == 0u) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (uint32_t k = 0; k < blockDim.x / 32u; ++k) tot += part[k];
    const float inv = 1.0f / sqrtf(tot / (float)n + eps);
    if (on) {
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint16_t o0 = f32_to_bf16_bits(f[2 * j] * inv * __uint_as_float(ww[j] << 16));
            const uint16_t o1 = f32_to_bf16_bits(f[2 * j + 1] * inv * __uint_as_float(ww[j] & 0xFFFF0000u));
            o[j] = (uint32_t)o0 | ((uint32_t)o1 << 16);
        }
        reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * n)[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (advance != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *advance = *advance + 1u;
}

// Tagged gathered buffer -> plain bf16 [rows, cols]: the operand form the tensor-core GEMM's TMA loads need.
__global__ void detag_rows_kernel(const TaggedIn tin, uint16_t* __restrict__ out, uint32_t cols) {
    pdl_trigger();
    pdl_wait();
    const uint32_t tag = (*tin.step - 1u) * tin.layers + tin.lsel;
    const uint64_t* tr = tin.words + (size_t)blockIdx.y * tin.pitch;
    uint32_t* orow = reinterpret_cast<uint32_t*>(out + (size_t)blockIdx.y * cols);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < cols / 2u; i += gridDim.x * blockDim.x)
        orow[i] = ld_tagged_pair(tr + i, tag, tin);
}

}  // namespace mcl

mc_status_t mcl::residual_rmsnorm_rows_tagged(uint16_t* d_res, const uint16_t* d_add, const uint16_t* d_norm_w, uint16_t* d_out,
                                              uint32_t rows, uint32_t n, float eps, const TaggedIn& add, uint32_t* d_advance,
                                              cudaStream_t stream, bool pdl) {
    if (add.words != nullptr && (n & 1u) != 0u) { set_error("residual_rmsnorm_rows: a tagged addend needs an even width"); return MC_E_INVALID_ARGUMENT; }
    const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0u; };
    const bool vec = (n & 7u) == 0u && n <= 8192u && al16(d_res) && al16(d_norm_w) && al16(d_out) &&
                     (add.words != nullptr || al16(d_add));
    if (vec) (void)launch(residual_rmsnorm_rows_vec_kernel, dim3(rows), dim3((n / 8u + 31u) / 32u * 32u), 0, stream, pdl, d_res, d_add, d_norm_w, d_out, n, eps, add, d_advance);
    else (void)launch(residual_rmsnorm_rows_kernel, dim3(rows), dim3(256), 0, stream, pdl, d_res, d_add, d_norm_w, d_out, n, eps, add, d_advance);
    MCL_CHECK_LAUNCH("residual_rmsnorm_rows");
    return MC_OK;
}

mc_status_t mcl::detag_rows(const TaggedIn& in, uint16_t* d_out, uint32_t rows, uint32_t cols, cudaStream_t stream, bool pdl) {
    if (in.words == nullptr || d_out == nullptr || rows == 0 || cols == 0 || (cols & 1u) != 0u) { set_error("detag_rows: invalid args"); return MC_E_INVALID_ARGUMENT; }
    const uint32_t gx = (cols / 2u + 255u) / 256u;
    (void)launch(detag_rows_kernel, dim3(gx < 16u ? gx : 16u, rows), dim3(256), 0, stream, pdl, in, d_out, cols);
    MCL_CHECK_LAUNCH("detag_rows");
    return MC_OK;
}

using namespace mcl;

// =======================================================================================
// extern "C"
// =======================================================================================
extern "C" {

const char* mc_sm100_last_error(void) { return g_err; }

// Debug hook (not part of the frozen surface, like the reference's mc_debug_*):
// selects the math form per weight type; -1 keeps the current one.
void mc_sm100_debug_set_math(int32_t bf16_math, int32_t fp8_math) {
    if (bf16_math >= 0 && bf16_math <= 2) g_math[2].store(bf16_math);
    if (fp8_math >= 0 && fp8_math <= 2) g_math[1].store(fp8_math);
}

int32_t mc_sm100_debug_take_error(void) { return skinny_take_error(); }

void mc_sm100_debug_set_mma_rows(int32_t max_m) { mma_rows_set_max_m(max_m); }

// Host-only views of two launch plans (no CUDA call), for tests of the host logic.
void mc_sm100_debug_mma_rows_plan(uint32_t N, uint32_t sms, uint32_t* rows, uint32_t* blocks_at_a_time, uint32_t* worst_rows) {
    const MmaRowsPlan p = mma_rows_plan(N, sms == 0u ? 148u : sms);
    if (rows) *rows = p.rows;
    if (blocks_at_a_time) *blocks_at_a_time = p.r;
    if (worst_rows) *worst_rows = p.worst_rows;
}
void mc_sm100_debug_chain_plan(int32_t fp8, uint32_t hidden, uint32_t inter, uint32_t* slot_bytes, uint32_t* rows_hidden,
                               uint32_t* rows_gate_up, uint32_t* rows_down) {
    const int wb = fp8 ? 1 : 2;
    const uint32_t kmax = hidden > inter ? hidden : inter;
    const uint32_t unit_max = (2u * hidden > inter ? 2u * hidden : inter) * (uint32_t)wb;
    const uint32_t slot = chain_slot_bytes(wb, hidden, kmax, unit_max);
    if (slot_bytes) *slot_bytes = slot;
    if (rows_hidden) *rows_hidden = slot ? chain_rows_per_unit(wb, hidden, EPI_STORE, slot) : 0u;
    if (rows_gate_up) *rows_gate_up = slot ? chain_rows_per_unit(wb, hidden, EPI_SWIGLU, slot) : 0u;
    if (rows_down) *rows_down = slot ? chain_rows_per_unit(wb, inter, EPI_STORE, slot) : 0u;
}

void mc_sm100_hint_next_weights(const void* d_next_w, uint64_t bytes) {
    g_next = (d_next_w != nullptr && aligned16(d_next_w) && bytes >= 16u) ? NextWeights{d_next_w, bytes & ~(uint64_t)15u}
                                                                          : NextWeights{nullptr, 0};
}

void mc_sm100_debug_set_prefetch(int32_t mode, int32_t chunk_bytes, int32_t evict_first, int64_t cap_bytes) {
    if (mode >= 0 && mode <= 2) g_pf_mode.store((uint32_t)mode);
    if (chunk_bytes >= 128 && chunk_bytes <= (1 << 20)) g_pf_chunk.store((uint32_t)chunk_bytes & ~127u);
    if (evict_first >= 0) g_pf_evict_first.store(evict_first ? 1u : 0u);
    if (cap_bytes > 0) g_pf_cap.store((uint64_t)cap_bytes);
}

// Host-only check of the per-device shared-memory opt-in bookkeeping (no CUDA call is made): returns 0, or the
// number of the expectation that failed.
int32_t mc_sm100_debug_optin_selftest(void) {
    static SmemOptIn o;                       // zero-initialised
    std::atomic<int> raised[kMaxDevices];
    for (auto& r : raised) r.store(0);
    auto on = [&](int dev, size_t bytes, cudaError_t result = cudaSuccess) {
        return o.ensure_on(dev, bytes, [&] { raised[dev].fetch_add(1); return result; });
    };
    if (on(0, 40u * 1024u) != cudaSuccess || raised[0] != 0) return 1;          // below 48 KB: nothing to raise
    if (on(0, 100u * 1024u) != cudaSuccess || raised[0] != 1) return 2;         // first use on device 0
    if (on(0, 100u * 1024u) != cudaSuccess || raised[0] != 1) return 3;         // remembered
    if (on(0, 64u * 1024u) != cudaSuccess || raised[0] != 1) return 4;          // a smaller request is covered
    if (on(1, 100u * 1024u) != cudaSuccess || raised[1] != 1) return 5;         // another device: raised again
    if (on(0, 200u * 1024u) != cudaSuccess || raised[0] != 2) return 6;         // a larger request raises again
    if (on(63, 100u * 1024u) != cudaSuccess || raised[63] != 1) return 7;
    if (on(64, 100u * 1024u) != cudaErrorInvalidDevice || on(-1, 100u * 1024u) != cudaErrorInvalidDevice) return 8;
    if (on(2, 100u * 1024u, cudaErrorInvalidValue) != cudaErrorInvalidValue || o.recorded(2) != 0u) return 9;   // a failed raise is not remembered
    if (on(2, 100u * 1024u) != cudaSuccess || raised[2] != 2) return 10;
    // host threads racing for one device: exactly one raise
    std::thread th[8];
    for (auto& t : th) t = std::thread([&] { for (int i = 0; i < 1000; ++i) (void)on(5, 150u * 1024u); });
    for (auto& t : th) t.join();
    if (raised[5] != 1 || o.recorded(5) != 150u * 1024u) return 11;
    return 0;
}

mc_status_t mc_sm100_device_check(int32_t* out_sm_count, uint64_t* out_l2_bytes,
                                  int32_t* out_cc_major, int32_t* out_cc_minor) {
    clear_error();
    int dev = 0, major = 0, minor = 0, sms = 0, l2 = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
    if (e != cudaSuccess) {
        set_error("device query failed: %s", cudaGetErrorString(e));
        return MC_E_CUDA;
    }
    if (out_sm_count) *out_sm_count = sms;
    if (out_l2_bytes) *out_l2_bytes = (uint64_t)l2;
    if (out_cc_major) *out_cc_major = major;
    if (out_cc_minor) *out_cc_minor = minor;
    if (major != 10) {
        set_error("device %d is compute capability %d.%d; this library is built for 10.x (sm_100a)", dev,
                  major, minor);
        return MC_E_UNSUPPORTED;
    }
    return MC_OK;
}

mc_status_t mc_sm100_decode_gemv(const uint16_t* d_w, const uint16_t* d_x, uint16_t* d_y, uint32_t N,
                                 uint32_t K, int32_t tactic, uint32_t split_s, float* d_split_partial,
                                 void* stream, int32_t pdl) {
    clear_error();
    if (d_w == nullptr || d_x == nullptr || d_y == nullptr || N == 0 || K == 0 || (K & 7u) != 0 ||
        !aligned16(d_w) || !aligned16(d_x)) {
        set_error("mc_sm100_decode_gemv: invalid args (N=%u K=%u tactic=%d)", N, K, tactic);
        return MC_E_INVALID_ARGUMENT;
    }
    RowsArgs a{};
    a.w = d_w; a.x = d_x; a.y = d_y; a.N = N; a.K = K; a.y_stride = N; a.kseg = K;
    const cudaStream_t st = (cudaStream_t)stream;
    if (tactic == MC_GEMV_TACTIC_ROWS) return rows(2, 1, PRO_NONE, EPI_STORE, a, 1, st, pdl != 0);
    if (tactic == MC_GEMV_TACTIC_SPLITK) {
        if (d_split_partial == nullptr || split_s < 2u || K % split_s != 0u || (K / split_s) % 8u != 0u) {
            set_error("mc_sm100_decode_gemv: bad split-K config (S=%u K=%u partial=%p)", split_s, K,
                      (const void*)d_split_partial);
            return MC_E_INVALID_ARGUMENT;
        }
        a.kseg = K / split_s;
        a.partial = d_split_partial;
        const mc_status_t s = rows(2, 1, PRO_NONE, EPI_PARTIAL, a, split_s, st, pdl != 0);
        if (s != MC_OK) return s;
        (void)launch(splitk_merge_kernel, dim3((N + 255u) / 256u), dim3(256), 0, st, pdl != 0,
                     (const float*)d_split_partial, (const float*)nullptr, split_s, N, N, d_y);
        MCL_CHECK_LAUNCH("splitk_merge");
        return MC_OK;
    }
    set_error("mc_sm100_decode_gemv: unknown tactic %d (library GEMM tactic 0 does not exist here)", tactic);
    return MC_E_INVALID_ARGUMENT;
}

static mc_status_t fp8_rows_any(const uint8_t* d_w, const float* d_scale, const uint16_t* d_x,
                                uint16_t* d_y, uint32_t M, uint32_t N, uint32_t K, cudaStream_t st,
                                bool pdl) {
    if ((K & 15u) == 0u && aligned16(d_w) && aligned16(d_x)) {
        RowsArgs a{};
        a.w = d_w; a.scale = d_scale; a.x = d_x; a.y = d_y; a.N = N; a.K = K; a.y_stride = N; a.kseg = K;
        return rows(1, (int)M, PRO_NONE, EPI_STORE, a, 1, st, pdl);
    }
    (void)launch(gemv_fp8_bytes_kernel, dim3((N + 7u) / 8u), dim3(256), 0, st, pdl, d_w, d_scale, d_x, d_y,
                 M, N, K);
    MCL_CHECK_LAUNCH("gemv_fp8_bytes");
    return MC_OK;
}

mc_status_t mc_sm100_gemv_fp8(const uint8_t* d_w, const float* d_scale, const uint16_t* d_x,
                              uint16_t* d_y, uint32_t N, uint32_t K, void* stream, int32_t pdl) {
    clear_error();
    if (d_w == nullptr || d_scale == nullptr || d_x == nullptr || d_y == nullptr || N == 0 || K == 0) {
        set_error("mc_sm100_gemv_fp8: invalid args (N=%u K=%u)", N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    return fp8_rows_any(d_w, d_scale, d_x, d_y, 1, N, K, (cudaStream_t)stream, pdl != 0);
}

static mc_status_t prologue_common(int wb, const void* d_w, const float* d_scale, const uint16_t* d_res_in,
                                   const uint16_t* d_addend, const uint16_t* d_norm_w,
                                   uint16_t* d_res_out, uint16_t* d_y, uint32_t N, uint32_t n, float eps,
                                   void* stream, int32_t pdl, const char* who) {
    clear_error();
    if (d_w == nullptr || (wb == 1 && d_scale == nullptr) || d_res_in == nullptr || d_norm_w == nullptr ||
        d_res_out == nullptr || d_y == nullptr || N == 0 || n == 0 || (n % (wb == 2 ? 8u : 16u)) != 0 ||
        !aligned16(d_w) || d_res_in == d_res_out) {
        set_error("%s: invalid args (N=%u n=%u)", who, N, n);
        return MC_E_INVALID_ARGUMENT;
    }
    RowsArgs a{};
    a.w = d_w; a.scale = d_scale; a.y = d_y; a.N = N; a.K = n; a.y_stride = N; a.kseg = n;
    a.res_in = d_res_in; a.addend = d_addend; a.norm_w = d_norm_w; a.res_out = d_res_out; a.eps = eps;
    return rows(wb, 1, PRO_RESNORM, EPI_STORE, a, 1, (cudaStream_t)stream, pdl != 0);
}

mc_status_t mc_sm100_gemv_rows_prologue(const uint16_t* d_w, const uint16_t* d_res_in,
                                        const uint16_t* d_addend, const uint16_t* d_norm_w,
                                        uint16_t* d_res_out, uint16_t* d_y, uint32_t N, uint32_t n,
                                        float eps, void* stream, int32_t pdl) {
    return prologue_common(2, d_w, nullptr, d_res_in, d_addend, d_norm_w, d_res_out, d_y, N, n, eps, stream,
                           pdl, "mc_sm100_gemv_rows_prologue");
}

mc_status_t mc_sm100_gemv_fp8_prologue(const uint8_t* d_w, const float* d_scale, const uint16_t* d_res_in,
                                       const uint16_t* d_addend, const uint16_t* d_norm_w,
                                       uint16_t* d_res_out, uint16_t* d_y, uint32_t N, uint32_t n,
                                       float eps, void* stream, int32_t pdl) {
    return prologue_common(1, d_w, d_scale, d_res_in, d_addend, d_norm_w, d_res_out, d_y, N, n, eps, stream,
                           pdl, "mc_sm100_gemv_fp8_prologue");
}

static mc_status_t swiglu_in_common(int wb, const void* d_w, const float* d_scale,
                                    const uint16_t* d_gate_up, uint16_t* d_y, uint32_t N, uint32_t K,
                                    void* stream, int32_t pdl, const char* who) {
    clear_error();
    if (d_w == nullptr || (wb == 1 && d_scale == nullptr) || d_gate_up == nullptr || d_y == nullptr ||
        N == 0 || K == 0 || (K % (wb == 2 ? 8u : 16u)) != 0 || !aligned16(d_w)) {
        set_error("%s: invalid args (N=%u K=%u)", who, N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    RowsArgs a{};
    a.w = d_w; a.scale = d_scale; a.y = d_y; a.N = N; a.K = K; a.y_stride = N; a.kseg = K;
    a.gate_up = d_gate_up;
    return rows(wb, 1, PRO_SWIGLU, EPI_STORE, a, 1, (cudaStream_t)stream, pdl != 0);
}

mc_status_t mc_sm100_gemv_rows_swiglu(const uint16_t* d_w, const uint16_t* d_gate_up, uint16_t* d_y,
                                      uint32_t N, uint32_t K, void* stream, int32_t pdl) {
    return swiglu_in_common(2, d_w, nullptr, d_gate_up, d_y, N, K, stream, pdl, "mc_sm100_gemv_rows_swiglu");
}

mc_status_t mc_sm100_gemv_fp8_swiglu(const uint8_t* d_w, const float* d_scale, const uint16_t* d_gate_up,
                                     uint16_t* d_y, uint32_t N, uint32_t K, void* stream, int32_t pdl) {
    return swiglu_in_common(1, d_w, d_scale, d_gate_up, d_y, N, K, stream, pdl, "mc_sm100_gemv_fp8_swiglu");
}

mc_status_t mc_sm100_gate_up_swiglu(const void* d_w, const float* d_scale, const uint16_t* d_x,
                                    uint16_t* d_y, uint32_t M, uint32_t N, uint32_t K, void* stream,
                                    int32_t pdl) {
    clear_error();
    const int wb = d_scale == nullptr ? 2 : 1;
    if (d_w == nullptr || d_x == nullptr || d_y == nullptr || M == 0 || M > 64u || N == 0 || (N & 1u) != 0 ||
        K == 0 || (K % (wb == 2 ? 8u : 16u)) != 0 || !aligned16(d_w) || !aligned16(d_x)) {
        set_error("mc_sm100_gate_up_swiglu: invalid args (M=%u N=%u K=%u)", M, N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    if (M > 4u && wb == 2) return batched_linear_bf16(d_w, d_x, d_y, M, N, K, true, (cudaStream_t)stream, pdl != 0);
    if (M > 4u)
        return skinny_gemm(SKINNY_W_E4M3, d_w, d_scale, d_x, nullptr, d_y, M, N, K, true, (cudaStream_t)stream, pdl != 0);
    RowsArgs a{};
    a.w = d_w; a.scale = d_scale; a.x = d_x; a.y = d_y; a.N = N; a.K = K; a.y_stride = N / 2u; a.kseg = K;
    return rows(wb, (int)M, PRO_NONE, EPI_SWIGLU, a, 1, (cudaStream_t)stream, pdl != 0);
}

mc_status_t mc_sm100_gate_up_swiglu_prologue(const void* d_w, const float* d_scale, const uint16_t* d_res_in,
                                             const uint16_t* d_addend, const uint16_t* d_norm_w,
                                             uint16_t* d_res_out, uint16_t* d_y, uint32_t N, uint32_t n,
                                             float eps, void* stream, int32_t pdl) {
    clear_error();
    const int wb = d_scale == nullptr ? 2 : 1;
    if (d_w == nullptr || d_res_in == nullptr || d_norm_w == nullptr || d_res_out == nullptr ||
        d_y == nullptr || N == 0 || (N & 1u) != 0 || n == 0 || (n % (wb == 2 ? 8u : 16u)) != 0 ||
        !aligned16(d_w) || d_res_in == d_res_out) {
        set_error("mc_sm100_gate_up_swiglu_prologue: invalid args (N=%u n=%u)", N, n);
        return MC_E_INVALID_ARGUMENT;
    }
    RowsArgs a{};
    a.w = d_w; a.scale = d_scale; a.y = d_y; a.N = N; a.K = n; a.y_stride = N / 2u; a.kseg = n;
    a.res_in = d_res_in; a.addend = d_addend; a.norm_w = d_norm_w; a.res_out = d_res_out; a.eps = eps;
    return rows(wb, 1, PRO_RESNORM, EPI_SWIGLU, a, 1, (cudaStream_t)stream, pdl != 0);
}

mc_status_t mc_sm100_interleave_rows(const void* d_src, void* d_dst, uint32_t I, uint32_t row_bytes,
                                     void* stream) {
    clear_error();
    if (d_src == nullptr || d_dst == nullptr || d_src == d_dst || I == 0 || row_bytes == 0) {
        set_error("mc_sm100_interleave_rows: invalid args (I=%u row_bytes=%u)", I, row_bytes);
        return MC_E_INVALID_ARGUMENT;
    }
    interleave_rows_kernel<<<dim3(2u * I), dim3(128), 0, (cudaStream_t)stream>>>(
        (const uint8_t*)d_src, (uint8_t*)d_dst, I, row_bytes);
    MCL_CHECK_LAUNCH("interleave_rows");
    return MC_OK;
}

// ---- batched ------------------------------------------------------------------------

mc_status_t mc_sm100_gemv_fp8_rows_m(const uint8_t* d_w, const float* d_scale, const uint16_t* d_x,
                                     uint16_t* d_y, uint32_t M, uint32_t N, uint32_t K, void* stream,
                                     int32_t pdl) {
    clear_error();
    if (d_w == nullptr || d_scale == nullptr || d_x == nullptr || d_y == nullptr || M < 2u || M > 64u ||
        N == 0 || K == 0) {
        set_error("mc_sm100_gemv_fp8_rows_m: invalid args (M=%u N=%u K=%u)", M, N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    const cudaStream_t st = (cudaStream_t)stream;
    if (M <= 3u || !skinny_shape_ok(N, K, 1)) {
        // CUDA cores up to three rows (each row then bit-equal to the M = 1 call of the same form; four rows
        // cost 14.4 us on the down_proj shape against 11.1 us on the tensor cores); rows beyond are served
        // four at a time (only shapes tcgen05 cannot take get here with M > 3).
        for (uint32_t m0 = 0; m0 < M; m0 += 4u) {
            const uint32_t mc = M - m0 < 4u ? M - m0 : 4u;
            const mc_status_t s = fp8_rows_any(d_w, d_scale, d_x + (size_t)m0 * K, d_y + (size_t)m0 * N, mc,
                                               N, K, st, pdl != 0);
            if (s != MC_OK) return s;
        }
        return MC_OK;
    }
    return skinny_gemm(SKINNY_W_E4M3, d_w, d_scale, d_x, nullptr, d_y, M, N, K, false, st, pdl != 0);
}

size_t mc_sm100_gemm_workspace_bytes(uint32_t M, uint32_t N, uint32_t K) {
    return skinny_workspace_bytes(M, N, K);
}

mc_status_t mc_sm100_gemm_bf16(void* stream, void* d_workspace, size_t ws_size, uint32_t M, uint32_t N,
                               uint32_t K, const void* d_a, const void* d_b, void* d_c) {
    clear_error();
    if (d_a == nullptr || d_b == nullptr || d_c == nullptr || M == 0 || M > 64u || N == 0 || K == 0 ||
        (K & 7u) != 0 || !aligned16(d_a) || !aligned16(d_b)) {
        set_error("mc_sm100_gemm_bf16: invalid args (M=%u N=%u K=%u)", M, N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    const cudaStream_t st = (cudaStream_t)stream;
    // one row: the streaming GEMV; two and more: the tensor-core kernel (measured on the down_proj shape,
    // M = 2 / 4: 9.3 / 10.8 us on CUDA cores against 8.8 us), CUDA cores only for shapes it cannot take
    if (M < 2u || !skinny_shape_ok(N, K, 2)) {
        for (uint32_t m0 = 0; m0 < M; m0 += 4u) {
            const uint32_t mc = M - m0 < 4u ? M - m0 : 4u;
            RowsArgs a{};
            a.w = d_a; a.x = (const uint16_t*)d_b + (size_t)m0 * K; a.y = (uint16_t*)d_c + (size_t)m0 * N;
            a.N = N; a.K = K; a.y_stride = N; a.kseg = K;
            const mc_status_t s = rows(2, (int)mc, PRO_NONE, EPI_STORE, a, 1, st, false);
            if (s != MC_OK) return s;
        }
        return MC_OK;
    }
    (void)d_workspace;
    (void)ws_size;
    // launched with the programmatic-dependent-launch attribute: the kernel prefetches only
    // weights before griddepcontrol.wait, so this is equivalent to plain stream order
    return batched_linear_bf16(d_a, (const uint16_t*)d_b, (uint16_t*)d_c, M, N, K, false, st, true);
}

mc_status_t mc_sm100_gemm_fp8_q(void* stream, void* d_workspace, size_t ws_size, uint32_t M, uint32_t N,
                                uint32_t K, const void* d_w_fp8, const float* d_w_scale,
                                const void* d_x_fp8, const float* d_x_scale, uint16_t* d_y_bf16) {
    clear_error();
    if (d_w_fp8 == nullptr || d_w_scale == nullptr || d_x_fp8 == nullptr || d_x_scale == nullptr ||
        d_y_bf16 == nullptr || M == 0 || M > 64u || N == 0 || K == 0 || (K & 15u) != 0 ||
        !aligned16(d_w_fp8) || !aligned16(d_x_fp8)) {
        set_error("mc_sm100_gemm_fp8_q: invalid args (M=%u N=%u K=%u)", M, N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    if (!skinny_shape_ok(N, K, 1)) {
        set_error("mc_sm100_gemm_fp8_q: shape N=%u K=%u not supported by the tcgen05 path", N, K);
        return MC_E_UNSUPPORTED;
    }
    (void)d_workspace;
    (void)ws_size;
    return skinny_gemm(SKINNY_W8A8, d_w_fp8, d_w_scale, (const uint16_t*)d_x_fp8, d_x_scale, d_y_bf16, M, N, K, false,
                       (cudaStream_t)stream, true);
}

mc_status_t mc_sm100_quant_rows(const uint16_t* d_x, uint8_t* d_xq, float* d_scale, uint32_t M, uint32_t K,
                                void* stream) {
    clear_error();
    if (d_x == nullptr || d_xq == nullptr || d_scale == nullptr || M == 0 || K == 0) {
        set_error("mc_sm100_quant_rows: invalid args (M=%u K=%u)", M, K);
        return MC_E_INVALID_ARGUMENT;
    }
    quant_rows_kernel<<<dim3(M < 1024u ? M : 1024u), dim3(256), 0, (cudaStream_t)stream>>>(d_x, d_xq, d_scale,
                                                                                         M, K);
    MCL_CHECK_LAUNCH("quant_rows");
    return MC_OK;
}

mc_status_t mc_sm100_post_scale_rows(uint16_t* d_y, const float* d_w_scale, const float* d_x_scale,
                                     uint32_t M, uint32_t N, void* stream) {
    clear_error();
    if (d_y == nullptr || d_w_scale == nullptr || M == 0 || N == 0) {
        set_error("mc_sm100_post_scale_rows: invalid args (M=%u N=%u)", M, N);
        return MC_E_INVALID_ARGUMENT;
    }
    const size_t tot = (size_t)M * N;
    const uint32_t blocks = (uint32_t)((tot + 255u) / 256u < 4096u ? (tot + 255u) / 256u : 4096u);
    post_scale_rows_kernel<<<dim3(blocks), dim3(256), 0, (cudaStream_t)stream>>>(d_y, d_w_scale, d_x_scale, M,
                                                                                  N);
    MCL_CHECK_LAUNCH("post_scale_rows");
    return MC_OK;
}

mc_status_t mc_sm100_gemm_fp8(void* stream, void* d_workspace, size_t ws_size, uint32_t M, uint32_t N,
                              uint32_t K, const void* d_w_fp8, const float* d_w_scale,
                              const uint16_t* d_x_bf16, uint16_t* d_y_bf16, void* d_x_fp8_scratch,
                              float* d_x_scale_scratch) {
    clear_error();
    if (d_x_bf16 == nullptr || d_x_fp8_scratch == nullptr || d_x_scale_scratch == nullptr) {
        set_error("mc_sm100_gemm_fp8: invalid args (M=%u N=%u K=%u)", M, N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    const mc_status_t s = mc_sm100_quant_rows(d_x_bf16, (uint8_t*)d_x_fp8_scratch, d_x_scale_scratch, M, K, stream);
    if (s != MC_OK) return s;
    return mc_sm100_gemm_fp8_q(stream, d_workspace, ws_size, M, N, K, d_w_fp8, d_w_scale, d_x_fp8_scratch,
                               d_x_scale_scratch, d_y_bf16);
}

mc_status_t mc_sm100_residual_rmsnorm_rows(uint16_t* d_res, const uint16_t* d_add, const uint16_t* d_norm_w,
                                           uint16_t* d_out, uint32_t rows, uint32_t n, float eps, void* stream,
                                           int32_t pdl) {
    clear_error();
    if (d_res == nullptr || d_norm_w == nullptr || d_out == nullptr || rows == 0 || n == 0) {
        set_error("mc_sm100_residual_rmsnorm_rows: invalid args (rows=%u n=%u)", rows, n);
        return MC_E_INVALID_ARGUMENT;
    }
    return residual_rmsnorm_rows_tagged(d_res, d_add, d_norm_w, d_out, rows, n, eps, TaggedIn{}, nullptr, (cudaStream_t)stream, pdl != 0);
}

// ---- greedy -------------------------------------------------------------------------

size_t mc_sm100_argmax_stage_bytes(uint32_t n_rows) {
    // room for either producer: 64 slices per row (standalone) or up to 1024
    // CTA candidates per row (fused lm_head epilogue); value + index each.
    return (size_t)(n_rows ? n_rows : 1u) * 1024u * (sizeof(float) + sizeof(int32_t));
}

static void stage_split(void* d_stage, uint32_t n_rows, float** v, int32_t** i) {
    *v = (float*)d_stage;
    *i = (int32_t*)((uint8_t*)d_stage + (size_t)n_rows * 1024u * sizeof(float));
}

mc_status_t mc_sm100_argmax_bf16(const uint16_t* d_logits, uint32_t n_rows, uint32_t vocab,
                                 uint32_t row_stride, int32_t index_base, void* d_stage,
                                 int32_t* d_out_idx, float* d_out_val, void* stream, int32_t pdl) {
    clear_error();
    if (d_logits == nullptr || d_stage == nullptr || d_out_idx == nullptr || n_rows == 0 || vocab == 0 ||
        row_stride < vocab) {
        set_error("mc_sm100_argmax_bf16: invalid args (rows=%u vocab=%u stride=%u)", n_rows, vocab, row_stride);
        return MC_E_INVALID_ARGUMENT;
    }
    float* sv;
    int32_t* si;
    stage_split(d_stage, n_rows, &sv, &si);
    const cudaStream_t st = (cudaStream_t)stream;
    (void)launch(argmax_stage1_kernel, dim3(kArgmaxSlices, n_rows), dim3(kArgmaxThreads), 0, st, pdl != 0,
                 d_logits, vocab, row_stride, index_base, sv, si);
    MCL_CHECK_LAUNCH("argmax_stage1");
    (void)launch(argmax_stage2_kernel, dim3(n_rows), dim3(64), 0, st, pdl != 0, (const float*)sv,
                 (const int32_t*)si, kArgmaxSlices, n_rows, 1, d_out_idx, d_out_val);
    MCL_CHECK_LAUNCH("argmax_stage2");
    return MC_OK;
}

mc_status_t mc_sm100_lm_head_argmax(const void* d_w, const float* d_scale, const uint16_t* d_x,
                                    uint16_t* d_logits, uint32_t y_stride, uint32_t M, uint32_t N,
                                    uint32_t K, int32_t index_base, void* d_stage, int32_t* d_out_idx,
                                    float* d_out_val, void* stream, int32_t pdl) {
    clear_error();
    const int wb = d_scale == nullptr ? 2 : 1;
    if (d_w == nullptr || d_x == nullptr || d_logits == nullptr || d_stage == nullptr ||
        d_out_idx == nullptr || M == 0 || M > 8u || N == 0 || K == 0 || y_stride < N ||
        (K % (wb == 2 ? 8u : 16u)) != 0 || !aligned16(d_w) || !aligned16(d_x)) {
        set_error("mc_sm100_lm_head_argmax: invalid args (M=%u N=%u K=%u stride=%u)", M, N, K, y_stride);
        return MC_E_INVALID_ARGUMENT;
    }
    const cudaStream_t st = (cudaStream_t)stream;
    float* sv;
    int32_t* si;
    stage_split(d_stage, M, &sv, &si);
    if (M <= 4u) {
        RowsArgs a{};
        a.w = d_w; a.scale = d_scale; a.x = d_x; a.y = d_logits; a.N = N; a.K = K; a.y_stride = y_stride;
        a.kseg = K; a.stage_val = sv; a.stage_idx = si; a.index_base = index_base;
        const mc_status_t s = rows(wb, (int)M, PRO_NONE, EPI_ARGMAX, a, 1, st, pdl != 0);
        if (s != MC_OK) return s;
        // candidates: kArgmaxCands slots laid out [slot][m]
        (void)launch(argmax_stage2_kernel, dim3(M), dim3(256), 0, st, pdl != 0, (const float*)sv,
                     (const int32_t*)si, kArgmaxCands, M, 0, d_out_idx, d_out_val);
        MCL_CHECK_LAUNCH("argmax_stage2");
        return MC_OK;
    }
    // 5..8 rows: batched GEMM, then the standalone two-stage argmax on its logits.
    mc_status_t s;
    if (wb == 2) {
        if (y_stride != N) {
            set_error("mc_sm100_lm_head_argmax: M > 4 needs y_stride == N");
            return MC_E_UNSUPPORTED;
        }
        s = mc_sm100_gemm_bf16(stream, nullptr, 0, M, N, K, d_w, d_x, d_logits);
    } else {
        if (y_stride != N) {
            set_error("mc_sm100_lm_head_argmax: M > 4 needs y_stride == N");
            return MC_E_UNSUPPORTED;
        }
        s = mc_sm100_gemv_fp8_rows_m((const uint8_t*)d_w, d_scale, d_x, d_logits, M, N, K, stream, pdl);
    }
    if (s != MC_OK) return s;
    return mc_sm100_argmax_bf16(d_logits, M, N, y_stride, index_base, d_stage, d_out_idx, d_out_val, stream, pdl);
}

static mc_status_t lm_head_prologue_impl(const char* who, const void* d_w, const float* d_scale, const uint16_t* d_res_in,
                                         const uint16_t* d_addend, const uint16_t* d_norm_w, uint16_t* d_res_out,
                                         uint16_t* d_logits, uint32_t N, uint32_t n, float eps, int32_t index_base,
                                         void* d_stage, int32_t* d_out_idx, float* d_out_val,
                                         const mc_sm100_shard_io_t* io, void* stream, int32_t pdl) {
    const int wb = d_scale == nullptr ? 2 : 1;
    if (d_w == nullptr || d_res_in == nullptr || d_norm_w == nullptr || d_res_out == nullptr ||
        d_logits == nullptr || d_stage == nullptr || d_out_idx == nullptr || N == 0 || n == 0 ||
        (n % (wb == 2 ? 8u : 16u)) != 0 || !aligned16(d_w) || d_res_in == d_res_out) {
        set_error("%s: invalid args (N=%u n=%u)", who, N, n);
        return MC_E_INVALID_ARGUMENT;
    }
    const cudaStream_t st = (cudaStream_t)stream;
    float* sv;
    int32_t* si;
    stage_split(d_stage, 1, &sv, &si);
    RowsArgs a{};
    a.w = d_w; a.scale = d_scale; a.y = d_logits; a.N = N; a.K = n; a.y_stride = N; a.kseg = n;
    a.res_in = d_res_in; a.addend = d_addend; a.norm_w = d_norm_w; a.res_out = d_res_out; a.eps = eps;
    a.stage_val = sv; a.stage_idx = si; a.index_base = index_base;
    mc_status_t s;
    if (io != nullptr) {
        // the addend is a tagged vector gathered from all ranks: only the decode-chain kernel reads those
        s = shard_io_to_args(who, io, N, false, a.sh);
        if (s != MC_OK) return s;
        const NextWeights nw = take_next_weights();
        a.pf.ptr = static_cast<const uint8_t*>(nw.ptr); a.pf.bytes = nw.bytes;
        s = wb == 2 ? launch_fast<2>(PRO_RESNORM, EPI_ARGMAX, a, st, pdl != 0) : launch_fast<1>(PRO_RESNORM, EPI_ARGMAX, a, st, pdl != 0);
    } else {
        s = rows(wb, 1, PRO_RESNORM, EPI_ARGMAX, a, 1, st, pdl != 0);
    }
    if (s != MC_OK) return s;
    (void)launch(argmax_stage2_kernel, dim3(1), dim3(256), 0, st, pdl != 0, (const float*)sv,
                 (const int32_t*)si, kArgmaxCands, 1u, 0, d_out_idx, d_out_val);
    MCL_CHECK_LAUNCH("argmax_stage2");
    return MC_OK;
}

mc_status_t mc_sm100_lm_head_argmax_prologue(const void* d_w, const float* d_scale, const uint16_t* d_res_in,
                                             const uint16_t* d_addend, const uint16_t* d_norm_w,
                                             uint16_t* d_res_out, uint16_t* d_logits, uint32_t N, uint32_t n,
                                             float eps, int32_t index_base, void* d_stage,
                                             int32_t* d_out_idx, float* d_out_val, void* stream,
                                             int32_t pdl) {
    clear_error();
    return lm_head_prologue_impl("mc_sm100_lm_head_argmax_prologue", d_w, d_scale, d_res_in, d_addend, d_norm_w, d_res_out,
                                 d_logits, N, n, eps, index_base, d_stage, d_out_idx, d_out_val, nullptr, stream, pdl);
}

mc_status_t mc_sm100_lm_head_argmax_sharded(const void* d_w, const float* d_scale, const uint16_t* d_res_in,
                                            const uint16_t* d_addend, const uint16_t* d_norm_w,
                                            uint16_t* d_res_out, uint16_t* d_logits, uint32_t N, uint32_t n,
                                            float eps, int32_t index_base, void* d_stage, int32_t* d_out_idx,
                                            float* d_out_val, const mc_sm100_shard_io_t* io, void* stream,
                                            int32_t pdl) {
    clear_error();
    if (io == nullptr) { set_error("mc_sm100_lm_head_argmax_sharded: no exchange descriptor"); return MC_E_INVALID_ARGUMENT; }
    return lm_head_prologue_impl("mc_sm100_lm_head_argmax_sharded", d_w, d_scale, d_res_in, d_addend, d_norm_w, d_res_out,
                                 d_logits, N, n, eps, index_base, d_stage, d_out_idx, d_out_val, io, stream, pdl);
}

// ---- host-buffer convenience -----------------------------------------------------------

mc_status_t mc_sm100_linear_host(int32_t kind, const void* d_w, const float* d_scale, const uint16_t* h_x,
                                 uint16_t* h_y, uint32_t M, uint32_t N, uint32_t K, uint16_t* d_x_stage,
                                 uint16_t* d_y_stage, void* d_workspace, size_t ws_size, void* stream) {
    clear_error();
    if (h_x == nullptr || h_y == nullptr || d_x_stage == nullptr || d_y_stage == nullptr || M == 0 || N == 0 ||
        K == 0 || (kind != 0 && kind != 1)) {
        set_error("mc_sm100_linear_host: invalid args (kind=%d M=%u N=%u K=%u)", kind, M, N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    const cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(d_x_stage, h_x, (size_t)M * K * 2u, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) {
        set_error("mc_sm100_linear_host: H2D failed: %s", cudaGetErrorString(e));
        return MC_E_CUDA;
    }
    mc_status_t s;
    uint32_t n_out = N;
    if (kind == 1) {
        s = mc_sm100_gate_up_swiglu(d_w, d_scale, d_x_stage, d_y_stage, M, N, K, stream, 0);
        n_out = N / 2u;
    } else if (d_scale == nullptr) {
        s = M == 1 ? mc_sm100_decode_gemv((const uint16_t*)d_w, d_x_stage, d_y_stage, N, K, MC_GEMV_TACTIC_ROWS, 0,
                                          nullptr, stream, 0)
                   : mc_sm100_gemm_bf16(stream, d_workspace, ws_size, M, N, K, d_w, d_x_stage, d_y_stage);
    } else {
        s = M == 1 ? mc_sm100_gemv_fp8((const uint8_t*)d_w, d_scale, d_x_stage, d_y_stage, N, K, stream, 0)
                   : mc_sm100_gemv_fp8_rows_m((const uint8_t*)d_w, d_scale, d_x_stage, d_y_stage, M, N, K,
                                              stream, 0);
    }
    if (s != MC_OK) return s;
    e = cudaMemcpyAsync(h_y, d_y_stage, (size_t)M * n_out * 2u, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        set_error("mc_sm100_linear_host: D2H/sync failed: %s", cudaGetErrorString(e));
        return MC_E_CUDA;
    }
    return MC_OK;
}

}  // extern "C"
