// gemm_mma_rows.cu -- batched-decode GEMM for 2 <= M <= 16 rows, bf16 weights, streamed through registers.
//
// The tcgen05 kernel (skinny_gemm.cu) pays ~4 us per call on top of its HBM time at these batch sizes: a
// tensor-map pipeline through shared memory, one (row tile, K slice) per CTA and a cluster reduction over
// eight K slices, because 128-row tiles leave a 2304-row matrix with 18 of them.  At M <= 16 the activation
// is a few KB, and what has to move is the weights -- exactly the M = 1 problem.  So this kernel is the M = 1
// streaming GEMV with a real B operand:
//   * the weight's blocks of 16 (or 8) rows are dealt to the CTAs as contiguous, near-equal ranges; a CTA works
//     on R blocks of its range at a time and the 16 / R warps of a block take its 32-element K steps round-robin
//     (they read adjacent 64-byte pieces of every row).  R = blocks per CTA when that is at most 16 (one pass,
//     e.g. gate_up: 5 blocks x 3 warps; qkv: 3 blocks of 8 rows x 5 warps; down: 1 block x 16 warps), else 16
//     (a warp owns whole blocks: long streams, nothing to add up across warps);
//   * lane (g, t) loads 16 bytes of row g and of row 8 + g per step with 128-bit streaming loads -- straight
//     into mma.sync.m16n8k16 A fragments: the mma's k index is only a labelling, and the B fragment, 16 bytes
//     of activation row g at the SAME k offset, is cut up the same way; four steps are in flight per warp in
//     each of two register buffers, the first before griddepcontrol.wait.  The B fragments come straight from
//     L2 (every CTA reads the M x K activation exactly once, spread over its K steps);
//   * fp32 accumulators D[16 x 8] per 8 activation rows; the 16 warps' partial tiles meet in shared memory
//     and are added in warp order (bit-reproducible), then scaled / SwiGLU'd / rounded / stored -- or, in a
//     sharded step, sent to every rank's gathered buffer as tagged words like the tcgen05 epilogue does.
// No shared-memory staging of weights, no tensor map, no cluster.  Where it wins and where it does not: see the
// measurements above batched_linear_bf16 at the end of this file.
#include "gemm_mma_rows.cuh"

#include "gemv_fast.cuh"
#include "skinny_gemm.cuh"

#include <atomic>

namespace mcl {

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kU = 4;            // K steps per register buffer

struct MmaRowsArgs {
    const uint16_t* w;
    const uint16_t* x;
    uint16_t* y;
    uint32_t M, N, K, x_pitch, swiglu;
    uint32_t kw, r;         // warps that share one row block; row blocks a CTA holds at a time (r * kw <= 16)
    PeerOut out;
};

__device__ __forceinline__ uint4 ld_l2_16(const void* p) {      // activations another kernel wrote: read at L2
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

}  // namespace

// MB: 8-row blocks of the activation (M <= 8 MB).  ROWS: weight rows per block, 16 or 8 (8: the upper half of
// every A fragment is zero; chosen when it spreads the blocks more evenly over the SMs).
template <int MB, int ROWS>
__global__ void __launch_bounds__(kThreads, 1) gemm_mma_rows_kernel(const MmaRowsArgs a) {
    __shared__ __align__(16) float part[kWarps][16][8 * MB];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t K = a.K, N = a.N, M = a.M;
    const uint32_t S = K / 32u;                                   // K steps of 32 elements
    const uint32_t KW = a.kw, R = a.r, kwi = warp % KW, slot = warp / KW;        // slot >= R: a warp without work
    const uint32_t my_steps = slot < R && S > kwi ? (S - kwi + KW - 1u) / KW : 0u;
    const uint32_t nb = ((S + KW - 1u) / KW + kU - 1u) / kU;      // batches per row block, the same for every warp
    const uint32_t nblk = (N + ROWS - 1u) / ROWS;
    const uint32_t blk_lo = (uint32_t)((uint64_t)nblk * blockIdx.x / gridDim.x), blk_hi = (uint32_t)((uint64_t)nblk * (blockIdx.x + 1u) / gridDim.x);
    const uint32_t passes = (blk_hi - blk_lo + R - 1u) / R;
    const uint32_t T = passes * nb;                               // batches this warp walks through
    const uint64_t policy = l2_policy_stream(true);

    uint4 rawA[kU][2], rawB[kU][2];
    auto issue = [&](uint4 (&raw)[kU][2], uint32_t q) {
        const uint32_t rb = blk_lo + (q / nb) * R + slot, i0 = (q % nb) * kU;
        const uint32_t r0 = rb * ROWS + g;
        const bool mine = rb < blk_hi;
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const uint32_t i = i0 + (uint32_t)u;
            const uint32_t koff = 32u * (kwi + KW * i) + 8u * t;
            const bool in = mine && i < my_steps;
            raw[u][0] = in && r0 < N ? ld_stream16_hint(a.w + (size_t)r0 * K + koff, policy) : make_uint4(0u, 0u, 0u, 0u);
            if constexpr (ROWS == 16)
                raw[u][1] = in && r0 + 8u < N ? ld_stream16_hint(a.w + (size_t)(r0 + 8u) * K + koff, policy) : make_uint4(0u, 0u, 0u, 0u);
            else
                raw[u][1] = make_uint4(0u, 0u, 0u, 0u);
        }
    };
    float2 d01[MB], d23[MB];
    auto zero = [&]() {
#pragma unroll
        for (int c = 0; c < MB; ++c) { d01[c] = make_float2(0.f, 0.f); d23[c] = make_float2(0.f, 0.f); }
    };
    auto consume = [&](uint4 (&raw)[kU][2], uint32_t q) {
        const uint32_t i0 = (q % nb) * kU;
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const uint32_t i = i0 + (uint32_t)u;
            const uint32_t koff = 32u * (kwi + KW * i) + 8u * t;
            const bool in = i < my_steps;            // beyond: zero weights against zero activations
#pragma unroll
            for (int c = 0; c < MB; ++c) {
                const uint32_t m = 8u * (uint32_t)c + g;
                const uint4 xf = in && m < M ? ld_l2_16(a.x + (size_t)m * a.x_pitch + koff) : make_uint4(0u, 0u, 0u, 0u);
                mma16816_bf16(d01[c], d23[c], raw[u][0].x, raw[u][1].x, raw[u][0].y, raw[u][1].y, xf.x, xf.y);
                mma16816_bf16(d01[c], d23[c], raw[u][0].z, raw[u][1].z, raw[u][0].w, raw[u][1].w, xf.z, xf.w);
            }
        }
    };
    // the R row blocks are done: the warps' partial tiles -> shared memory -> each block's tiles summed in warp
    // order -> epilogue
    auto flush = [&](uint32_t q) {
#pragma unroll
        for (int c = 0; c < MB; ++c) {
            *reinterpret_cast<float2*>(&part[warp][g][8 * c + 2 * t]) = d01[c];
            *reinterpret_cast<float2*>(&part[warp][g + 8][8 * c + 2 * t]) = d23[c];
        }
        zero();
        __syncthreads();
        const uint64_t out_tag = a.out.world != 0u ? (uint64_t)((*a.out.step - 1u) * a.out.layers + a.out.lsel) << 32 : 0ull;
        auto put_pair = [&](uint32_t m, uint32_t c, uint16_t v0, uint16_t v1) {       // output columns c (even), c + 1 of row m
            const uint64_t word = out_tag | ((uint64_t)v1 << 16) | (uint64_t)v0;
            for (uint32_t p = 0; p < a.out.world; ++p)
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;"
                             ::"l"(reinterpret_cast<uint64_t*>(a.out.base[p]) + (size_t)m * a.out.pitch + a.out.col0 + (c >> 1)), "l"(word) : "memory");
        };
        // per block: PER work items (one output, or one pair of outputs); item -> (block slot, index within the block)
        const uint32_t per = a.out.world == 0u ? (a.swiglu ? 8u * 8u * MB : 16u * 8u * MB) : (a.swiglu ? 4u * 8u * MB : 8u * 8u * MB);
        for (uint32_t idx = tid; idx < R * per; idx += kThreads) {
            const uint32_t sl = idx / per, e = idx % per;
            const uint32_t rb = blk_lo + (q / nb) * R + sl, row0 = rb * ROWS;
            if (rb >= blk_hi) continue;
            auto tile = [&](uint32_t i, uint32_t m) {
                float acc = 0.f;
                for (uint32_t w = sl * KW; w < (sl + 1u) * KW; ++w) acc += part[w][i][m];
                return acc;
            };
            auto swi = [&](uint32_t i, uint32_t m) {      // SwiGLU of weight rows i (gate), i + 1 (up) of the block
                const float gt = __uint_as_float((uint32_t)f32_to_bf16_bits(tile(i, m)) << 16);
                const float up = __uint_as_float((uint32_t)f32_to_bf16_bits(tile(i + 1u, m)) << 16);
                return f32_to_bf16_bits(swiglu_f32(gt, up));
            };
            if (a.out.world == 0u) {
                if (!a.swiglu) {
                    const uint32_t i = e & 15u, m = e >> 4;           // rows fastest: 32-byte runs per activation row
                    if (i < (uint32_t)ROWS && row0 + i < N && m < M) a.y[(size_t)m * N + row0 + i] = f32_to_bf16_bits(tile(i, m));
                } else {
                    const uint32_t j = e & 7u, m = e >> 3;
                    if (2u * j < (uint32_t)ROWS && row0 + 2u * j + 1u < N && m < M) a.y[(size_t)m * (N / 2u) + (row0 >> 1) + j] = swi(2u * j, m);
                }
            } else if (!a.swiglu) {
                const uint32_t p = e & 7u, m = e >> 3, i = 2u * p;    // output columns row0 + i, row0 + i + 1
                if (i < (uint32_t)ROWS && row0 + i < N && m < M)
                    put_pair(m, row0 + i, f32_to_bf16_bits(tile(i, m)), row0 + i + 1u < N ? f32_to_bf16_bits(tile(i + 1u, m)) : (uint16_t)0);
            } else {
                const uint32_t p = e & 3u, m = e >> 2, i = 4u * p;    // output columns (row0 + i) / 2 and the next one
                if (i < (uint32_t)ROWS && row0 + i + 1u < N && m < M)
                    put_pair(m, (row0 + i) >> 1, swi(i, m), row0 + i + 3u < N ? swi(i + 2u, m) : (uint16_t)0);
            }
        }
        __syncthreads();
    };

    if (T > 0u) issue(rawA, 0u);
    pdl_trigger();
    pdl_wait();
    zero();
    uint32_t q = 0;
    while (q < T) {
        if (q + 1u < T) issue(rawB, q + 1u);
        consume(rawA, q);
        if (q % nb == nb - 1u) flush(q);
        if (++q >= T) break;
        if (q + 1u < T) issue(rawA, q + 1u);
        consume(rawB, q);
        if (q % nb == nb - 1u) flush(q);
        ++q;
    }
}

// ---- host side ---------------------------------------------------------------------------

// Block height (16 or 8 rows) and blocks a CTA holds at a time (R): the height that leaves the fullest SM with fewer
// rows (16 on a tie); R = the most blocks any CTA owns, at most 16.
MmaRowsPlan mma_rows_plan(uint32_t N) { return mma_rows_plan(N, (uint32_t)sm_count()); }

MmaRowsPlan mma_rows_plan(uint32_t N, uint32_t sms) {
    MmaRowsPlan best{};
    for (uint32_t rows : {16u, 8u}) {
        const uint32_t blocks = (N + rows - 1u) / rows, grid = blocks < sms ? blocks : sms;
        const uint32_t per = (blocks + grid - 1u) / grid;          // the most blocks a CTA owns
        const uint32_t worst = per * rows;
        if (best.rows == 0u || worst < best.worst_rows)
            best = MmaRowsPlan{rows, per < (uint32_t)kWarps ? per : (uint32_t)kWarps, blocks, worst, 0.f};
    }
    best.balance = (float)N / (float)(best.blocks < sms ? best.blocks : sms) / (float)best.worst_rows;
    return best;
}

bool mma_rows_ok(uint32_t M, uint32_t N, uint32_t K, const void* w, const void* x, uint32_t x_pitch) {
    if (x_pitch == 0u) x_pitch = K;
    return M >= 2u && M <= 16u && N > 0u && K >= 32u && (K & 31u) == 0u && aligned16(w) && aligned16(x) && (x_pitch & 7u) == 0u && x_pitch >= K;
}

mc_status_t gemm_mma_rows(const void* w, const uint16_t* x, uint16_t* y, uint32_t M, uint32_t N, uint32_t K, bool swiglu,
                          cudaStream_t stream, bool pdl, uint32_t x_pitch, const PeerOut* out) {
    if (x_pitch == 0u) x_pitch = K;
    if (!mma_rows_ok(M, N, K, w, x, x_pitch) || (swiglu && (N & 1u)) || (out != nullptr && ((swiglu ? N / 2u : N) & 1u))) {
        set_error("gemm_mma_rows: invalid args (M=%u N=%u K=%u x_pitch=%u)", M, N, K, x_pitch);
        return MC_E_INVALID_ARGUMENT;
    }
    MmaRowsArgs a{};
    a.w = reinterpret_cast<const uint16_t*>(w); a.x = x; a.y = y;
    a.M = M; a.N = N; a.K = K; a.x_pitch = x_pitch; a.swiglu = swiglu ? 1u : 0u;
    if (out != nullptr) a.out = *out;
    (void)take_next_weights();          // a hint left for this launch is consumed (this kernel does no L2 prefetch)
    const bool two = M > 8u;
    const MmaRowsPlan pl = mma_rows_plan(N);
    const bool half = pl.rows == 8u;
    a.r = pl.r;
    a.kw = (uint32_t)kWarps / pl.r;
    const uint32_t sms = (uint32_t)sm_count();
    const dim3 grid(pl.blocks < sms ? pl.blocks : sms), block(kThreads);
    if (half) {
        if (two) (void)launch(gemm_mma_rows_kernel<2, 8>, grid, block, 0, stream, pdl, a);
        else (void)launch(gemm_mma_rows_kernel<1, 8>, grid, block, 0, stream, pdl, a);
    } else {
        if (two) (void)launch(gemm_mma_rows_kernel<2, 16>, grid, block, 0, stream, pdl, a);
        else (void)launch(gemm_mma_rows_kernel<1, 16>, grid, block, 0, stream, pdl, a);
    }
    MCL_CHECK_LAUNCH("gemm_mma_rows");
    return MC_OK;
}

// Measured on B200 (us per call in a chain, this kernel / tcgen05 kernel): down 2304 x 5760 M = 2: 6.9 / 8.6, M = 8: 7.3 / 8.6,
// M = 16: 9.2 / 8.7; o 2304 x 2304 M = 8: 3.9 / 4.9; but qkv 3456 x 2304 M = 8: 7.7 / 6.0, gate_up 11520 x 2304 M = 8: 14.3 / 12.2,
// lm_head M = 8: 148 / 103 (staging the activation in shared memory instead: 7.0, 12.9, 113, and down 9.0, o 5.4; eight
// warps and two CTAs per SM: down 10.3).  So the public batched entry points use it where a CTA owns a single row block
// (N <= 16 x SMs) and M <= 8.  The decode stack does not: there these linears sit between tcgen05 kernels of two CTAs
// per SM, beside which this one-CTA-per-SM kernel cannot become resident early (M = 8 step 2.11 ms against 1.91 ms).
static std::atomic<int> g_max_m{8};
void mma_rows_set_max_m(int max_m) { g_max_m.store(max_m < 0 ? 0 : (max_m > 16 ? 16 : max_m), std::memory_order_relaxed); }

mc_status_t batched_linear_bf16(const void* w, const uint16_t* x, uint16_t* y, uint32_t M, uint32_t N, uint32_t K, bool swiglu,
                                cudaStream_t stream, bool pdl, uint32_t x_pitch, const PeerOut* out) {
    if ((int)M <= g_max_m.load(std::memory_order_relaxed) && mma_rows_ok(M, N, K, w, x, x_pitch) && mma_rows_plan(N).r == 1u)
        return gemm_mma_rows(w, x, y, M, N, K, swiglu, stream, pdl, x_pitch, out);
    return skinny_gemm(SKINNY_W_BF16, w, nullptr, x, nullptr, y, M, N, K, swiglu, stream, pdl, x_pitch, out);
}

}  // namespace mcl
