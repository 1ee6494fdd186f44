// gemv_rows.cuh -- the CUDA-core streaming GEMV family for M <= 4 activation rows.
//
// One kernel template covers the bandwidth-bound linear layers of a decode
// step: bf16 or e4m3 weights, 1..4 activation rows, an optional prologue that
// builds the activation on chip (residual add + RMSNorm, or SwiGLU of a
// gate|up vector) and an epilogue that is a plain store, a SwiGLU over
// interleaved gate/up rows, a store + running argmax, or a split-K partial.
//
// Data movement: the weight matrix is streamed exactly once with 128-bit
// read-only loads that bypass L1; a warp owns R consecutive output rows and
// its lanes stride K in 16-byte units, so every load instruction of a warp
// covers R contiguous 512-byte runs.  A warp keeps R*U such loads in flight
// (the first batch is issued before griddepcontrol.wait, i.e. while the
// producer kernel is still draining).  The activation lives in shared memory
// as bf16 and is read with conflict-free 128-bit loads at the same unit index
// as the weights.  Row groups are dealt to CTAs round-robin and, inside a CTA,
// to warps round-robin, so every SM gets the same number of rows to within
// one group whatever N is.
//
// Arithmetic: fp32 accumulation of exact products, one rounding to bf16 at the
// end.  e4m3 weights are widened in registers; the per-row scale multiplies
// the finished sum once.  No floating-point atomics anywhere: results are
// bit-reproducible from run to run and between eager and graph replay.
#pragma once

#include "common.cuh"

namespace mcl {

enum : int { PRO_NONE = 0, PRO_RESNORM = 1, PRO_SWIGLU = 2 };
enum : int { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_ARGMAX = 2, EPI_PARTIAL = 3 };
enum : int { MATH_CVT = 0, MATH_MIXED = 1 };

// Candidates per logits row in the argmax stage buffer ([kArgmaxCands][M]).
constexpr uint32_t kArgmaxCands = 1024;

struct RowsArgs {
    const void* w;         // [N,K] bf16 bits or e4m3 codes, row-major
    const float* scale;    // [N] fp32 row scales (e4m3 only)
    const uint16_t* x;     // [M,K] bf16 (PRO_NONE)
    uint16_t* y;           // [M, y_stride] bf16
    float* partial;        // EPI_PARTIAL: [S, M, N] fp32
    uint32_t N, K, y_stride;
    uint32_t kseg;         // K elements handled by one blockIdx.y (== K unless split)
    // PRO_RESNORM
    const uint16_t* res_in;
    const uint16_t* addend;
    const uint16_t* norm_w;
    uint16_t* res_out;
    float eps;
    // PRO_SWIGLU: gate|up vector of 2K bf16
    const uint16_t* gate_up;
    // EPI_ARGMAX: per-CTA (value, index) candidates, [gridDim.x, M]
    float* stage_val;
    int32_t* stage_idx;
    int32_t index_base;
    // N-sharded exchange with peer GPUs (gemv_fast_kernel only; all zero = off)
    ShardIO sh;
    // L2 prefetch of the next kernel's weights (all zero = off); gemv_fast_kernel also takes the
    // eviction policy of its own loads from here
    PrefetchArgs pf;
};

// ---- per-unit multiply-accumulate -------------------------------------------------
// One 16-byte unit of weights against the matching activation elements.
// bf16: 8 elements, activation in one uint4.  e4m3: 16 elements, activation in
// two uint4.  Two independent chains (a0 even elements, a1 odd elements).
template <int MATH>
__device__ __forceinline__ void mac_unit_bf16(const uint4& w, const uint4& x, float& a0, float& a1) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
    const uint32_t xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if constexpr (MATH == MATH_MIXED) {
            fma_bf16(a0, (uint16_t)(wv[j] & 0xFFFFu), (uint16_t)(xv[j] & 0xFFFFu));
            fma_bf16(a1, (uint16_t)(wv[j] >> 16), (uint16_t)(xv[j] >> 16));
        } else {
            a0 = fmaf(bf16lo(wv[j]), bf16lo(xv[j]), a0);
            a1 = fmaf(bf16hi(wv[j]), bf16hi(xv[j]), a1);
        }
    }
}

template <int MATH>
__device__ __forceinline__ void mac_unit_fp8(const uint4& w, const uint4& xa, const uint4& xb,
                                             float& a0, float& a1) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
    const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if constexpr (MATH == MATH_MIXED) {
            const uint32_t p0 = e4m3x2_to_bf16x2_scaled<0x1404u>(wv[j]);  // codes 0,1
            const uint32_t p1 = e4m3x2_to_bf16x2_scaled<0x3424u>(wv[j]);  // codes 2,3
            fma_bf16(a0, (uint16_t)(p0 & 0xFFFFu), (uint16_t)(xv[2 * j] & 0xFFFFu));
            fma_bf16(a1, (uint16_t)(p0 >> 16), (uint16_t)(xv[2 * j] >> 16));
            fma_bf16(a0, (uint16_t)(p1 & 0xFFFFu), (uint16_t)(xv[2 * j + 1] & 0xFFFFu));
            fma_bf16(a1, (uint16_t)(p1 >> 16), (uint16_t)(xv[2 * j + 1] >> 16));
        } else {
            const float2 f0 = e4m3x2_to_f32x2((uint16_t)(wv[j] & 0xFFFFu));
            const float2 f1 = e4m3x2_to_f32x2((uint16_t)(wv[j] >> 16));
            a0 = fmaf(f0.x, bf16lo(xv[2 * j]), a0);
            a1 = fmaf(f0.y, bf16hi(xv[2 * j]), a1);
            a0 = fmaf(f1.x, bf16lo(xv[2 * j + 1]), a0);
            a1 = fmaf(f1.y, bf16hi(xv[2 * j + 1]), a1);
        }
    }
}

// Cold path of the hardware-conversion variant: decode by bit construction at
// true scale (codes 0x7F/0xFF -> +/-480), same chain assignment as the fast path.
__device__ __forceinline__ void mac_unit_fp8_bits(const uint4& w, const uint4& xa, const uint4& xb,
                                                  float& a0, float& a1) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
    const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        a0 = fmaf(e4m3_to_f32(wv[j] & 0xFFu), bf16lo(xv[2 * j]), a0);
        a1 = fmaf(e4m3_to_f32((wv[j] >> 8) & 0xFFu), bf16hi(xv[2 * j]), a1);
        a0 = fmaf(e4m3_to_f32((wv[j] >> 16) & 0xFFu), bf16lo(xv[2 * j + 1]), a0);
        a1 = fmaf(e4m3_to_f32(wv[j] >> 24), bf16hi(xv[2 * j + 1]), a1);
    }
}

// e4m3 codes 0x7F/0xFF are NaN for the hardware converter but +/-480 for the
// reference decoder; a unit that holds one takes the bit-construction path.
__device__ __forceinline__ bool has_nan_code(const uint4& w) {
    const uint32_t m = 0x7F7F7F7Fu, one = 0x01010101u, top = 0x80808080u;
    return ((((w.x & m) + one) | ((w.y & m) + one) | ((w.z & m) + one) | ((w.w & m) + one)) & top) != 0u;
}

// ---- the kernel --------------------------------------------------------------------
// WB: bytes per weight element (2 bf16, 1 e4m3).  M: activation rows.  R: output
// rows per warp per pass.  U: 16-byte loads per row kept in flight per lane.
template <int WB, int M, int R, int U, int PRO, int EPI, int MATH, int THREADS, int MINB>
__global__ void __launch_bounds__(THREADS, MINB) gemv_rows_kernel(const RowsArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem_raw);  // [M][kseg] bf16
    __shared__ float red_f[THREADS / 32][M > 1 ? M : 1];
    __shared__ int32_t red_i[THREADS / 32][M > 1 ? M : 1];

    constexpr int WPB = THREADS / 32;
    constexpr int EPV = 16 / WB;  // weight elements per 16-byte unit
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t klen = a.kseg;
    const uint32_t kbeg = blockIdx.y * klen;
    const uint32_t nvec = klen / EPV;
    const uint32_t groups = (a.N + R - 1) / R;
    const uint32_t gstep = WPB * gridDim.x;
    const size_t row_bytes = (size_t)a.K * WB;
    const uint8_t* wbase = reinterpret_cast<const uint8_t*>(a.w) + (size_t)kbeg * WB;

    uint4 wreg[R][U];
    auto issue = [&](uint32_t g, uint32_t i0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t row = g * R + r;
            const uint8_t* wr = wbase + (size_t)row * row_bytes;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t v = lane + 32u * (i0 + u);
                if (row < a.N && v < nvec) wreg[r][u] = ld_stream16(wr + (size_t)v * 16u);
                else wreg[r][u] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };

    uint32_t g = blockIdx.x + warp * gridDim.x;
    // Weights do not depend on the producer kernel: first batch goes out now.
    if (g < groups) issue(g, 0);
    prefetch_next_weights(a.pf, blockIdx.y * gridDim.x + blockIdx.x, threadIdx.x, THREADS);
    pdl_trigger();
    pdl_wait();

    // ---- activation into shared memory -------------------------------------------
    if constexpr (PRO == PRO_NONE) {
        const uint32_t nx = klen / 8u;  // uint4 units per activation row
        for (uint32_t i = threadIdx.x; i < nx * M; i += THREADS) {
            const uint32_t m = i / nx, c = i - m * nx;
            reinterpret_cast<uint4*>(xs)[i] =
                *reinterpret_cast<const uint4*>(a.x + (size_t)m * a.K + kbeg + c * 8u);
        }
    } else if constexpr (PRO == PRO_RESNORM) {
        // res = bf16(res_in + addend); the norm reads the ROUNDED residual.
        float ss = 0.f;
        for (uint32_t i = threadIdx.x; i < a.K; i += THREADS) {
            float r = __uint_as_float((uint32_t)a.res_in[i] << 16);
            uint16_t rb = a.res_in[i];
            if (a.addend != nullptr) {
                r += __uint_as_float((uint32_t)a.addend[i] << 16);
                rb = f32_to_bf16_bits(r);
                r = __uint_as_float((uint32_t)rb << 16);
            }
            xs[i] = rb;
            if (blockIdx.x == 0 && blockIdx.y == 0) a.res_out[i] = rb;
            ss = fmaf(r, r, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) red_f[warp][0] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < WPB; ++w) tot += red_f[w][0];  // fixed order
        const float inv = 1.0f / sqrtf(tot / (float)a.K + a.eps);
        for (uint32_t i = threadIdx.x; i < a.K; i += THREADS) {
            const float r = __uint_as_float((uint32_t)xs[i] << 16);
            const float nw = __uint_as_float((uint32_t)a.norm_w[i] << 16);
            xs[i] = f32_to_bf16_bits(r * inv * nw);
        }
    } else {  // PRO_SWIGLU
        for (uint32_t i = threadIdx.x; i < a.K; i += THREADS) {
            const float gt = __uint_as_float((uint32_t)a.gate_up[i] << 16);
            const float up = __uint_as_float((uint32_t)a.gate_up[a.K + i] << 16);
            xs[i] = f32_to_bf16_bits(swiglu_f32(gt, up));
        }
    }
    __syncthreads();

    float best_v[M];
    int32_t best_i[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { best_v[m] = -INFINITY; best_i[m] = INT32_MAX; }

    const uint32_t per_lane = (nvec + 31u) / 32u;  // units per lane, rounded up
    bool first = true;
    for (; g < groups; g += gstep) {
        float sc[R];
        if constexpr (WB == 1 && EPI != EPI_PARTIAL) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t row = g * R + r;
                sc[r] = row < a.N ? __ldg(a.scale + row) : 0.f;
            }
        }
        float acc0[R][M], acc1[R][M];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) { acc0[r][m] = 0.f; acc1[r][m] = 0.f; }

        for (uint32_t i0 = 0; i0 < per_lane; i0 += U) {
            if (!first) issue(g, i0);
            first = false;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t v = lane + 32u * (i0 + u);
                if (v < nvec) {
                    if constexpr (WB == 2) {
                        uint4 xq[M];
#pragma unroll
                        for (int m = 0; m < M; ++m)
                            xq[m] = reinterpret_cast<const uint4*>(xs + (size_t)m * klen)[v];
#pragma unroll
                        for (int r = 0; r < R; ++r)
#pragma unroll
                            for (int m = 0; m < M; ++m)
                                mac_unit_bf16<MATH>(wreg[r][u], xq[m], acc0[r][m], acc1[r][m]);
                    } else {
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            const uint4 xa = reinterpret_cast<const uint4*>(xs + (size_t)m * klen)[2 * v];
                            const uint4 xb = reinterpret_cast<const uint4*>(xs + (size_t)m * klen)[2 * v + 1];
#pragma unroll
                            for (int r = 0; r < R; ++r) {
                                if (MATH == MATH_CVT && has_nan_code(wreg[r][u]))
                                    mac_unit_fp8_bits(wreg[r][u], xa, xb, acc0[r][m], acc1[r][m]);
                                else
                                    mac_unit_fp8<MATH>(wreg[r][u], xa, xb, acc0[r][m], acc1[r][m]);
                            }
                        }
                    }
                }
            }
        }

        // ---- reduce and store ------------------------------------------------------
        float tot[R][M];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float s = warp_sum(acc0[r][m] + acc1[r][m]);
                if constexpr (WB == 1 && MATH == MATH_MIXED) s *= MCL_E4M3_UNSCALE;
                if constexpr (WB == 1 && EPI != EPI_PARTIAL) s *= sc[r];
                tot[r][m] = s;
            }
        if (lane == 0) {
            if constexpr (EPI == EPI_SWIGLU) {
                static_assert(EPI != EPI_SWIGLU || (R % 2) == 0, "SwiGLU epilogue needs row pairs");
#pragma unroll
                for (int r = 0; r + 1 < R; r += 2) {
                    const uint32_t row = g * R + r;
                    if (row + 1 < a.N) {
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            const float gt = __uint_as_float((uint32_t)f32_to_bf16_bits(tot[r][m]) << 16);
                            const float up = __uint_as_float((uint32_t)f32_to_bf16_bits(tot[r + 1][m]) << 16);
                            a.y[(size_t)m * a.y_stride + (row >> 1)] = f32_to_bf16_bits(swiglu_f32(gt, up));
                        }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t row = g * R + r;
                    if (row < a.N) {
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            if constexpr (EPI == EPI_PARTIAL) {
                                a.partial[((size_t)blockIdx.y * M + m) * a.N + row] = tot[r][m];
                            } else {
                                const uint16_t yb = f32_to_bf16_bits(tot[r][m]);
                                a.y[(size_t)m * a.y_stride + row] = yb;
                                if constexpr (EPI == EPI_ARGMAX) {
                                    const float v = __uint_as_float((uint32_t)yb << 16);
                                    const int32_t idx = (int32_t)row + a.index_base;
                                    if (v > best_v[m] || (v == best_v[m] && idx < best_i[m])) {
                                        best_v[m] = v;
                                        best_i[m] = idx;
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
    }

    if constexpr (EPI == EPI_ARGMAX) {
        // The stage buffer always holds kArgmaxCands candidates per row; slots of
        // CTAs this launch does not have are neutralised by CTA 0.
        if (blockIdx.x == 0) {
            for (uint32_t c = gridDim.x * M + threadIdx.x; c < kArgmaxCands * M; c += THREADS) {
                a.stage_val[c] = -INFINITY;
                a.stage_idx[c] = INT32_MAX;
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < M; ++m) { red_f[warp][m] = best_v[m]; red_i[warp][m] = best_i[m]; }
        }
        __syncthreads();
        if (threadIdx.x < M) {
            const int m = threadIdx.x;
            float bv = red_f[0][m];
            int32_t bi = red_i[0][m];
            for (int w = 1; w < WPB; ++w) {
                const float v = red_f[w][m];
                const int32_t i = red_i[w][m];
                if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
            }
            a.stage_val[(size_t)blockIdx.x * M + m] = bv;
            a.stage_idx[(size_t)blockIdx.x * M + m] = bi;
        }
    }
}

}  // namespace mcl
