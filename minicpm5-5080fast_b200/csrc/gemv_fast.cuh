// gemv_fast.cuh -- the M = 1 streaming GEMV tuned for the decode chain.
//
// Measured on B200, a decode step is a chain of dependent kernels in which the
// weights of kernel i+1 can be in flight while kernel i still runs (programmatic
// dependent launch), but everything that needs the activation has to wait for
// griddepcontrol.wait.  What remains on the critical path after that wait is:
// staging x, the multiply-accumulates, the reduction and the store.  This kernel
// therefore (1) issues -- and, where registers allow, also widens -- its weights
// BEFORE the wait, (2) keeps the post-wait arithmetic as short as the ISA allows:
//   bf16 weights: fma.rn.f32.bf16 straight on the loaded halves against x staged
//                 as bf16 (one issue slot per element, half the shared-memory
//                 traffic of an fp32 copy of x; a packed f32x2 form was measured
//                 slower: it doubles the x traffic, which is what bounds the burst);
//   e4m3 weights: hardware cvt.rn.f16x2.e4m3x2 (exact), x staged as f16 after an
//                 exact scaling by 2^6, mixed-precision fma.rn.f32.f16 (one issue
//                 slot per element, no integer-pipe work -- the integer pipe runs
//                 at half rate on sm_100 and bounded the bit-placement form).
// Arithmetic contract unchanged: exact products, fp32 accumulation, the row scale
// on the finished sum, one rounding.  The f16 staging is used only when every
// activation element survives the f32 -> f16 -> f32 round trip exactly (checked
// per call with one __syncthreads_or); otherwise, and for any row whose sum comes
// out NaN (e4m3 codes 0x7F/0xFF, which the hardware converter maps to NaN but the
// reference decodes as +/-480), the row is recomputed with the bit-placement
// decoder against the bf16 copy of x.
#pragma once

#include "gemv_rows.cuh"

namespace mcl {

__device__ __forceinline__ void fma_f32x2(float2& acc, const float2 a, const float2 b) {
    unsigned long long A, B, C;
    asm("mov.b64 %0, {%1, %2};" : "=l"(A) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(B) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(C) : "f"(acc.x), "f"(acc.y));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(C) : "l"(A), "l"(B));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(acc.x), "=f"(acc.y) : "l"(C));
}

__device__ __forceinline__ void fma_f16(float& acc, uint16_t a, uint16_t b) {
    asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(a), "h"(b));
}

__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint16_t pair) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(pair));
    return h2;
}

// x * 2^6 as f16 bits; ok = the value survives the trip back unchanged.
__device__ __forceinline__ uint16_t x_to_f16_scaled(float x, bool& ok) {
    const float xs = x * 64.0f;
    uint16_t h;
    float back;
    asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(xs));
    asm("cvt.f32.f16 %0, %1;" : "=f"(back) : "h"(h));
    ok = (back == xs);
    return h;
}
constexpr float kF16Unscale = 0.015625f;   // 2^-6

// Weights of one 16-byte unit in the form the post-wait loop consumes.
template <int WB> struct WideUnit;
template <> struct WideUnit<2> { uint32_t p[4]; };    // 8 bf16, consumed as they are
template <> struct WideUnit<1> { uint32_t h[8]; };    // 16 e4m3 -> 8 f16 pairs

__device__ __forceinline__ void widen(const uint4& raw, WideUnit<2>& o) {
    o.p[0] = raw.x; o.p[1] = raw.y; o.p[2] = raw.z; o.p[3] = raw.w;
}
__device__ __forceinline__ void widen(const uint4& raw, WideUnit<1>& o) {
    const uint32_t v[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        o.h[2 * j] = cvt_e4m3x2_f16x2((uint16_t)(v[j] & 0xFFFFu));
        o.h[2 * j + 1] = cvt_e4m3x2_f16x2((uint16_t)(v[j] >> 16));
    }
}

// One unit against x.  bf16: x as 8 bf16 (xb + 8v).  e4m3: x as 16 f16 (xh + 16v).
__device__ __forceinline__ void mac_wide(const WideUnit<2>& w, const uint16_t* xb8, float2& a, float2& b) {
    const uint4 x0 = reinterpret_cast<const uint4*>(xb8)[0];
    const uint32_t xv[4] = {x0.x, x0.y, x0.z, x0.w};
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
        fma_bf16(a.x, (uint16_t)(w.p[j] & 0xFFFFu), (uint16_t)(xv[j] & 0xFFFFu));
        fma_bf16(a.y, (uint16_t)(w.p[j] >> 16), (uint16_t)(xv[j] >> 16));
        fma_bf16(b.x, (uint16_t)(w.p[j + 1] & 0xFFFFu), (uint16_t)(xv[j + 1] & 0xFFFFu));
        fma_bf16(b.y, (uint16_t)(w.p[j + 1] >> 16), (uint16_t)(xv[j + 1] >> 16));
    }
}
__device__ __forceinline__ void mac_wide(const WideUnit<1>& w, const uint16_t* xh, float2& a, float2& b) {
    const uint4 x0 = reinterpret_cast<const uint4*>(xh)[0], x1 = reinterpret_cast<const uint4*>(xh)[1];
    const uint32_t xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
        fma_f16(a.x, (uint16_t)(w.h[j] & 0xFFFFu), (uint16_t)(xv[j] & 0xFFFFu));
        fma_f16(a.y, (uint16_t)(w.h[j] >> 16), (uint16_t)(xv[j] >> 16));
        fma_f16(b.x, (uint16_t)(w.h[j + 1] & 0xFFFFu), (uint16_t)(xv[j + 1] & 0xFFFFu));
        fma_f16(b.y, (uint16_t)(w.h[j + 1] >> 16), (uint16_t)(xv[j + 1] >> 16));
    }
}

// ---- the multiply-accumulate on the tensor cores (mma.sync m16n8k16, fp32 accumulators) ----
// The post-wait burst on CUDA cores is bound by the integer pipe: fma.rn.f32.bf16 / .f16 take 16-bit
// operands and every one has to be cut out of its packed register first (4.1 thread instructions per
// weight, measured; halving the multiplies alone takes 40 us off the 1.1 ms step).  A warp-wide mma
// multiplies what the lanes already hold, in the layout they hold it: lane (g, t) = (lane / 4, lane % 4)
// supplies A row g (its own four weights of this mma: registers a0, a2) and B column g (the four
// matching activations: b0, b1), so D[g][g] is the dot product over the 16 elements of lane group g, and
// the diagonal of D, accumulated over all mmas, holds the eight groups' partial sums of the row.  A second
// weight row goes to A rows 8..15 (a1, a3) against the same B: its sums are D[8 + g][g].  The rest of D is
// cross terms nobody reads.  Products of bf16 / f16 are exact, accumulation is fp32.
// Measured on the 40-layer stream: bf16 1.097 -> 1.065 ms.  e4m3 does not gain (0.892 -> 0.900 - 0.910 ms, lm_head
// 53 -> 53 - 60 us: its bound is the hardware conversion of the codes, which stays), so it keeps the CUDA-core form.
template <int WB> constexpr bool kGemvMma = WB == 2;

__device__ __forceinline__ void mma16816_bf16(float2& d01, float2& d23, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d01.x), "+f"(d01.y), "+f"(d23.x), "+f"(d23.y)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816_f16(float2& d01, float2& d23, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d01.x), "+f"(d01.y), "+f"(d23.x), "+f"(d23.y)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// One 16-byte unit of row 0 (and of row 1 when given) against the matching activations; every lane of the
// warp takes part (a lane without a unit passes zeros).  Two accumulator sets (A, B) take alternate mmas, so
// that a row's chain of dependent mmas is half as long; each set: d01 = (D[g][2t], D[g][2t+1]), d23 the same
// for row 8 + g.
struct MmaAcc { float2 a01, a23, b01, b23; };
__device__ __forceinline__ void mac_mma(const WideUnit<2>& w0, const WideUnit<2>* w1, const uint4& x, MmaAcc& d) {
    mma16816_bf16(d.a01, d.a23, w0.p[0], w1 ? w1->p[0] : 0u, w0.p[1], w1 ? w1->p[1] : 0u, x.x, x.y);
    mma16816_bf16(d.b01, d.b23, w0.p[2], w1 ? w1->p[2] : 0u, w0.p[3], w1 ? w1->p[3] : 0u, x.z, x.w);
}
__device__ __forceinline__ void mac_mma(const WideUnit<1>& w0, const WideUnit<1>* w1, const uint4& xa, const uint4& xc, MmaAcc& d) {
    const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xc.x, xc.y, xc.z, xc.w};
#pragma unroll
    for (int i = 0; i < 4; i += 2) {
        mma16816_f16(d.a01, d.a23, w0.h[2 * i], w1 ? w1->h[2 * i] : 0u, w0.h[2 * i + 1], w1 ? w1->h[2 * i + 1] : 0u, xv[2 * i], xv[2 * i + 1]);
        mma16816_f16(d.b01, d.b23, w0.h[2 * i + 2], w1 ? w1->h[2 * i + 2] : 0u, w0.h[2 * i + 3], w1 ? w1->h[2 * i + 3] : 0u, xv[2 * i + 2], xv[2 * i + 3]);
    }
}
// a row's sum in this lane's share: row 0 from (a01, b01), row 1 from (a23, b23)
__device__ __forceinline__ float mma_row(const MmaAcc& d, int r, uint32_t lane);
// This lane's element of D's diagonal (0 unless the lane holds one): group g's sum sits in lane (g, g / 2).
__device__ __forceinline__ float mma_diag(const float2& d, uint32_t lane) {
    const uint32_t g = lane >> 2, t = lane & 3u;
    return t == (g >> 1) ? ((g & 1u) ? d.y : d.x) : 0.f;
}
__device__ __forceinline__ float mma_row(const MmaAcc& d, int r, uint32_t lane) {
    return r == 0 ? mma_diag(d.a01, lane) + mma_diag(d.b01, lane) : mma_diag(d.a23, lane) + mma_diag(d.b23, lane);
}

// Exact e4m3 row against the bf16 copy of x, weights re-read from global memory
// (cold path: range fallback and rows that hold a NaN code).  Warp-collective.
__device__ __forceinline__ float fp8_row_exact(const uint8_t* wrow, const uint16_t* xb, uint32_t nvec, uint32_t lane) {
    float a0 = 0.f, a1 = 0.f;
    for (uint32_t v = lane; v < nvec; v += 32u) {
        const uint4 w = ld_stream16(wrow + (size_t)v * 16u);
        const uint4 xa = reinterpret_cast<const uint4*>(xb)[2 * v], xc = reinterpret_cast<const uint4*>(xb)[2 * v + 1];
        mac_unit_fp8<MATH_MIXED>(w, xa, xc, a0, a1);
    }
    return warp_sum(a0 + a1) * MCL_E4M3_UNSCALE;
}


// ---- the kernel ------------------------------------------------------------------------
// Packs eight bf16-rounded activations into the shared-memory forms: the bf16 copy
// (both weight types) and, for e4m3 weights, the 2^6-scaled f16 copy.
template <int WB>
__device__ __forceinline__ void put_x8(uint16_t* xh, uint16_t* xb, uint32_t c, const uint16_t (&bits)[8], bool& inexact) {
    uint4 q;
    q.x = bits[0] | ((uint32_t)bits[1] << 16); q.y = bits[2] | ((uint32_t)bits[3] << 16);
    q.z = bits[4] | ((uint32_t)bits[5] << 16); q.w = bits[6] | ((uint32_t)bits[7] << 16);
    reinterpret_cast<uint4*>(xb)[c] = q;
    if constexpr (WB == 1) {
        uint16_t h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            bool ok;
            h[j] = x_to_f16_scaled(__uint_as_float((uint32_t)bits[j] << 16), ok);
            inexact |= !ok;
        }
        uint4 p;
        p.x = h[0] | ((uint32_t)h[1] << 16); p.y = h[2] | ((uint32_t)h[3] << 16);
        p.z = h[4] | ((uint32_t)h[5] << 16); p.w = h[6] | ((uint32_t)h[7] << 16);
        reinterpret_cast<uint4*>(xh)[c] = p;
    }
}

__device__ __forceinline__ void unpack8(const uint4& q, uint16_t (&bits)[8]) {
    const uint32_t v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { bits[2 * j] = (uint16_t)(v[j] & 0xFFFFu); bits[2 * j + 1] = (uint16_t)(v[j] >> 16); }
}

// WB 2 = bf16 weights, 1 = e4m3.  R rows per warp pass (2 only for the SwiGLU epilogue,
// whose pairs are adjacent rows).  U units per lane per batch.  PRE (e4m3 only): run the
// hardware conversion of the first batch before griddepcontrol.wait (twice the registers).
// DB: keep a second register buffer so that, when a warp walks several row groups, the
// next group's loads are issued before the current group's arithmetic.
// MINB: CTAs per SM the register budget is sized for.  With 2, the CTA of the NEXT kernel in a
// chain becomes resident beside this one and has its weights in flight while this one computes.
template <int WB, int R, int U, bool PRE, bool DB, int PRO, int EPI, int THREADS, int MINB = 1>
__global__ void __launch_bounds__(THREADS, MINB) gemv_fast_kernel(const RowsArgs a) {
    static_assert(EPI != EPI_PARTIAL, "split-K partials are produced by gemv_rows_kernel");
    static_assert(!(PRE && WB == 2), "bf16 weights are consumed as loaded");
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // shared memory: [e4m3 only: x as f16 [K]] | x as bf16 [K] | [RESNORM: fp32 residual [K]]
    const uint32_t K = a.K;
    uint16_t* xh = reinterpret_cast<uint16_t*>(smem_raw);
    uint16_t* xb = xh + (WB == 1 ? K : 0);
    float* tmp = reinterpret_cast<float*>(xb + K);
    __shared__ float red_f[THREADS / 32];
    __shared__ int32_t red_i[THREADS / 32];

    constexpr int WPB = THREADS / 32;
    constexpr int EPV = 16 / WB;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t nvec = K / EPV;
    const uint32_t groups = (a.N + R - 1) / R;
    const uint32_t gstep = WPB * gridDim.x;
    const size_t row_bytes = (size_t)K * WB;
    const uint8_t* wbase = reinterpret_cast<const uint8_t*>(a.w);
    const uint32_t per_lane = (nvec + 31u) / 32u;
    const bool one_batch = per_lane <= (uint32_t)U;   // a whole row fits one batch of loads

    const uint64_t policy = l2_policy_stream(a.pf.evict_first != 0u);
    uint4 rawA[R][U];
    uint4 rawB[DB ? R : 1][DB ? U : 1];
    WideUnit<WB> wide[PRE ? R : 1][PRE ? U : 1];
    // e4m3: the rows' scales travel with the rows' first batch of weights, so that the multiply at
    // the end of a group does not wait for a load of its own
    float scA[R], scB[R];
#pragma unroll
    for (int r = 0; r < R; ++r) { scA[r] = 1.f; scB[r] = 1.f; }
    auto issue = [&](auto& raw, float (&sc)[R], uint32_t g, uint32_t i0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t row = g * R + r;
            const uint8_t* wr = wbase + (size_t)row * row_bytes;
            if constexpr (WB == 1) {
                if (i0 == 0u && row < a.N) sc[r] = __ldg(a.scale + row);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t v = lane + 32u * (i0 + u);
                raw[r][u] = (row < a.N && v < nvec) ? ld_stream16_hint(wr + (size_t)v * 16u, policy) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };

    uint32_t g = blockIdx.x + warp * gridDim.x;
    if (g < groups) {
        issue(rawA, scA, g, 0);
        if constexpr (PRE) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int u = 0; u < U; ++u) widen(rawA[r][u], wide[r][u]);
        }
    }
    // this kernel's first loads are out: now ask for the next kernel's weights (HBM -> L2)
    prefetch_next_weights(a.pf, blockIdx.x, threadIdx.x, THREADS);
    // the norm weights do not depend on the producer kernel either: this thread's first chunk of them is
    // fetched now, which takes one L2 round trip out of the post-wait path of the prologue
    uint4 nw_first = make_uint4(0u, 0u, 0u, 0u);
    if constexpr (PRO == PRO_RESNORM) {
        if (threadIdx.x < K / 8u) nw_first = __ldg(reinterpret_cast<const uint4*>(a.norm_w) + threadIdx.x);
    }
    pdl_trigger();
    pdl_wait();
    // sharded run: the activation (or the addend of the prologue) is a vector gathered from all
    // ranks, one tagged 32-bit word per element; staging polls the words until they are current
    const bool tagged = a.sh.in_tagged != 0u;
    const uint32_t in_tag = tagged ? shard_tag(a.sh, a.sh.in_seq_mul, a.sh.in_seq_add) : 0u;

    // ---- activation: global -> (prologue) -> shared, eight elements per thread and step ----
    bool inexact = false;
    const uint32_t nchunk = K / 8u;
    if constexpr (PRO == PRO_NONE) {
        for (uint32_t c = threadIdx.x; c < nchunk; c += THREADS) {
            uint16_t bits[8];
            if (tagged) ld_tagged8(reinterpret_cast<const uint32_t*>(a.x) + 8u * c, in_tag, a.sh, bits);
            else unpack8(reinterpret_cast<const uint4*>(a.x)[c], bits);
            put_x8<WB>(xh, xb, c, bits, inexact);
        }
    } else if constexpr (PRO == PRO_RESNORM) {
        // res = bf16(res_in + addend); the norm reads the ROUNDED residual (rmsnorm.cu:144-154)
        float ss = 0.f;
        for (uint32_t c = threadIdx.x; c < nchunk; c += THREADS) {
            uint16_t rb[8], ad[8];
            unpack8(reinterpret_cast<const uint4*>(a.res_in)[c], rb);
            if (a.addend != nullptr) {
                if (tagged) ld_tagged8(reinterpret_cast<const uint32_t*>(a.addend) + 8u * c, in_tag, a.sh, ad);
                else unpack8(reinterpret_cast<const uint4*>(a.addend)[c], ad);
            }
            float rf[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float r = __uint_as_float((uint32_t)rb[j] << 16);
                if (a.addend != nullptr) {
                    r += __uint_as_float((uint32_t)ad[j] << 16);
                    rb[j] = f32_to_bf16_bits(r);
                    r = __uint_as_float((uint32_t)rb[j] << 16);
                }
                rf[j] = r;
                ss = fmaf(r, r, ss);
            }
            reinterpret_cast<float4*>(tmp)[2 * c] = make_float4(rf[0], rf[1], rf[2], rf[3]);
            reinterpret_cast<float4*>(tmp)[2 * c + 1] = make_float4(rf[4], rf[5], rf[6], rf[7]);
            if (blockIdx.x == 0) {
                uint4 q;
                q.x = rb[0] | ((uint32_t)rb[1] << 16); q.y = rb[2] | ((uint32_t)rb[3] << 16);
                q.z = rb[4] | ((uint32_t)rb[5] << 16); q.w = rb[6] | ((uint32_t)rb[7] << 16);
                reinterpret_cast<uint4*>(a.res_out)[c] = q;
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) red_f[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < WPB; ++w) tot += red_f[w];   // fixed order
        const float inv = 1.0f / sqrtf(tot / (float)K + a.eps);
        for (uint32_t c = threadIdx.x; c < nchunk; c += THREADS) {   // same thread, same chunks as pass 1
            uint16_t nw[8], bits[8];
            unpack8(c == threadIdx.x ? nw_first : reinterpret_cast<const uint4*>(a.norm_w)[c], nw);
            const float4 r0 = reinterpret_cast<const float4*>(tmp)[2 * c], r1 = reinterpret_cast<const float4*>(tmp)[2 * c + 1];
            const float rf[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) bits[j] = f32_to_bf16_bits(rf[j] * inv * __uint_as_float((uint32_t)nw[j] << 16));
            put_x8<WB>(xh, xb, c, bits, inexact);
        }
    } else {  // PRO_SWIGLU: x[k] = bf16( silu(gate_up[k]) * gate_up[K + k] )
        for (uint32_t c = threadIdx.x; c < nchunk; c += THREADS) {
            uint16_t gt[8], up[8], bits[8];
            unpack8(reinterpret_cast<const uint4*>(a.gate_up)[c], gt);
            unpack8(reinterpret_cast<const uint4*>(a.gate_up + K)[c], up);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                bits[j] = f32_to_bf16_bits(swiglu_f32(__uint_as_float((uint32_t)gt[j] << 16), __uint_as_float((uint32_t)up[j] << 16)));
            put_x8<WB>(xh, xb, c, bits, inexact);
        }
    }
    const bool fallback = __syncthreads_or(inexact ? 1 : 0) != 0;   // also the staging barrier

    float best_v = -INFINITY;
    int32_t best_i = INT32_MAX;
    // where the outputs go: y, or (sharded) slot `rank` of every rank's gathered vector as tagged
    // words, one destination rank per lane; logits of a sharded lm_head stay local
    const bool push = (EPI != EPI_ARGMAX) && a.sh.out_slot != 0u;
    const uint32_t ndst = push ? a.sh.world : 1u;
    uint32_t* wdst = reinterpret_cast<uint32_t*>(a.sh.out_peer[lane & 7u]) + (size_t)a.sh.rank * a.sh.out_slot;
    const uint32_t out_tag = push ? shard_tag(a.sh, a.sh.out_seq_mul, a.sh.out_seq_add) << 16 : 0u;
    auto put_y = [&](uint32_t i, uint16_t yb) {
        if (push) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(wdst + i), "r"(out_tag | (uint32_t)yb) : "memory");
        else a.y[i] = yb;
    };

    // multiply-accumulate one batch held in `raw` (or in `wide` when it was converted early)
    auto mac_batch = [&](auto& raw, bool use_wide, uint32_t i0, float2 (&acc_a)[R], float2 (&acc_b)[R]) {
        if constexpr (kGemvMma<WB>) {
            // tensor cores.  Lanes beyond the row's last unit hold zero weights and pass zero activations.
            static_assert(R <= 2, "an mma takes two weight rows");
            // accumulators of the running group: row 0 in (acc_a[0], acc_b[0]), row 1 in (acc_a[1], acc_b[1])
            MmaAcc md;
            md.a01 = acc_a[0]; md.b01 = acc_b[0];
            md.a23 = R == 2 ? acc_a[R - 1] : make_float2(0.f, 0.f); md.b23 = R == 2 ? acc_b[R - 1] : make_float2(0.f, 0.f);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t v = lane + 32u * (i0 + u);
                const bool in = v < nvec;
                WideUnit<WB> w0, w1;
                if (PRE && use_wide) {
                    w0 = wide[0][PRE ? u : 0];
                    if constexpr (R == 2) w1 = wide[PRE ? 1 : 0][PRE ? u : 0];
                } else {
                    widen(raw[0][u], w0);
                    if constexpr (R == 2) widen(raw[R - 1][u], w1);
                }
                if constexpr (WB == 2) {
                    const uint4 x = in ? reinterpret_cast<const uint4*>(xb)[v] : make_uint4(0u, 0u, 0u, 0u);
                    mac_mma(w0, R == 2 ? &w1 : nullptr, x, md);
                } else {
                    const uint4 xa = in ? reinterpret_cast<const uint4*>(xh)[2u * v] : make_uint4(0u, 0u, 0u, 0u);
                    const uint4 xc = in ? reinterpret_cast<const uint4*>(xh)[2u * v + 1u] : make_uint4(0u, 0u, 0u, 0u);
                    mac_mma(w0, R == 2 ? &w1 : nullptr, xa, xc, md);
                }
            }
            acc_a[0] = md.a01; acc_b[0] = md.b01;
            if constexpr (R == 2) { acc_a[R - 1] = md.a23; acc_b[R - 1] = md.b23; }
            return;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t v = lane + 32u * (i0 + u);
            if (v < nvec) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (PRE && use_wide) {
                        if constexpr (WB == 2) mac_wide(wide[PRE ? r : 0][PRE ? u : 0], xb + 8u * v, acc_a[r], acc_b[r]);
                        else mac_wide(wide[PRE ? r : 0][PRE ? u : 0], xh + 16u * v, acc_a[r], acc_b[r]);
                    } else {
                        WideUnit<WB> w;
                        widen(raw[r][u], w);
                        if constexpr (WB == 2) mac_wide(w, xb + 8u * v, acc_a[r], acc_b[r]);
                        else mac_wide(w, xh + 16u * v, acc_a[r], acc_b[r]);
                    }
                }
            }
        }
    };
    // reduce, scale, store one group
    auto finish = [&](uint32_t g, const float (&sc)[R], float2 (&acc_a)[R], float2 (&acc_b)[R]) {
        float tot[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float s = kGemvMma<WB> ? warp_sum(mma_diag(acc_a[r], lane) + mma_diag(acc_b[r], lane))
                               : warp_sum((acc_a[r].x + acc_a[r].y) + (acc_b[r].x + acc_b[r].y));
            if constexpr (WB == 1) {
                s *= kF16Unscale;
                const uint32_t row = g * R + r;
                if ((fallback || s != s) && row < a.N)    // warp-uniform: s is the same in every lane
                    s = fp8_row_exact(wbase + (size_t)row * row_bytes, xb, nvec, lane);
                s *= sc[r];
            }
            tot[r] = s;
        }
        if (lane < ndst) {      // the sums are the same in every lane
            if constexpr (EPI == EPI_SWIGLU) {
                static_assert(EPI != EPI_SWIGLU || R == 2, "SwiGLU epilogue works on row pairs");
                const uint32_t row = g * R;
                if (row + 1 < a.N) {
                    const float gt = __uint_as_float((uint32_t)f32_to_bf16_bits(tot[0]) << 16);
                    const float up = __uint_as_float((uint32_t)f32_to_bf16_bits(tot[R - 1]) << 16);
                    put_y(row >> 1, f32_to_bf16_bits(swiglu_f32(gt, up)));
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t row = g * R + r;
                    if (row < a.N) {
                        const uint16_t yb = f32_to_bf16_bits(tot[r]);
                        put_y(row, yb);
                        if constexpr (EPI == EPI_ARGMAX) {
                            const float v = __uint_as_float((uint32_t)yb << 16);
                            const int32_t idx = (int32_t)row + a.index_base;
                            if (v > best_v || (v == best_v && idx < best_i)) { best_v = v; best_i = idx; }
                        }
                    }
                }
            }
        }
    };
    auto zero = [&](float2 (&acc_a)[R], float2 (&acc_b)[R]) {
#pragma unroll
        for (int r = 0; r < R; ++r) { acc_a[r] = make_float2(0.f, 0.f); acc_b[r] = make_float2(0.f, 0.f); }
    };

    const bool skip_mac = (WB == 1) && fallback;   // every row goes through the exact path in finish()
    if (DB && one_batch) {
        // whole rows per batch: the next group's loads go out before this group's arithmetic
        if constexpr (DB) {
            bool use_wide = true;
            while (g < groups) {
                float2 acc_a[R], acc_b[R];
                uint32_t g2 = g + gstep;
                if (g2 < groups) issue(rawB, scB, g2, 0);
                zero(acc_a, acc_b);
                if (!skip_mac) mac_batch(rawA, use_wide, 0, acc_a, acc_b);
                use_wide = false;
                finish(g, scA, acc_a, acc_b);
                g = g2;
                if (g >= groups) break;
                g2 = g + gstep;
                if (g2 < groups) issue(rawA, scA, g2, 0);
                zero(acc_a, acc_b);
                if (!skip_mac) mac_batch(rawB, false, 0, acc_a, acc_b);
                finish(g, scB, acc_a, acc_b);
                g = g2;
            }
        }
    } else {
        bool first = true;
        for (; g < groups; g += gstep) {
            float2 acc_a[R], acc_b[R];
            zero(acc_a, acc_b);
            for (uint32_t i0 = 0; i0 < per_lane; i0 += U) {
                if (!first) issue(rawA, scA, g, i0);
                if (!skip_mac) mac_batch(rawA, first, i0, acc_a, acc_b);
                first = false;
            }
            finish(g, scA, acc_a, acc_b);
        }
    }

    if constexpr (EPI == EPI_ARGMAX) {
        if (blockIdx.x == 0) {
            for (uint32_t c = gridDim.x + threadIdx.x; c < kArgmaxCands; c += THREADS) {
                a.stage_val[c] = -INFINITY;
                a.stage_idx[c] = INT32_MAX;
            }
        }
        if (lane == 0) { red_f[warp] = best_v; red_i[warp] = best_i; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float bv = red_f[0];
            int32_t bi = red_i[0];
            for (int w = 1; w < WPB; ++w)
                if (red_f[w] > bv || (red_f[w] == bv && red_i[w] < bi)) { bv = red_f[w]; bi = red_i[w]; }
            a.stage_val[blockIdx.x] = bv;
            a.stage_idx[blockIdx.x] = bi;
        }
    }
}

}  // namespace mcl
