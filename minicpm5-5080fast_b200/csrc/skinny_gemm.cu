// skinny_gemm.cu -- batched-decode GEMM for 4 < M <= 64 on the 5th-generation tensor cores.
//
// Y[M,N] = X[M,K] . W[N,K]^T is computed "swapped": the weight tile is the MMA's A
// operand (128 rows of W = the MMA M dimension), the activation rows are the B
// operand (MMA N = M padded to 16/32/64), so one tcgen05.mma covers 128 output
// features for every batch row and the accumulator D[128 x Mpad] (fp32) lives in
// 16..64 TMEM columns.  The kernel is still bandwidth-bound (W is streamed once);
// the tensor core only removes the per-row FMA cost that caps the CUDA-core family.
//
// One CTA = one (row tile, K split) work item; two CTAs fit per SM.  Warps 0-7
// stream W (and the matching X slice) from global memory into a 4-stage shared
// memory ring in the canonical K-major 128-byte-swizzled layout, converting e4m3
// weights to bf16 on the way (weight-only form); warp 8 issues the MMAs and
// commits each stage back to the producers; warps 0-3 then read the accumulator
// with tcgen05.ld into shared memory.  Small N is split along K over a thread-block
// cluster (up to 8 CTAs per row tile): after a cluster barrier every CTA sums its
// slice of the tile over the cluster's partial accumulators through distributed
// shared memory, in rank order (no atomics, no global scratch, bit-reproducible),
// applies the scales (and the SwiGLU over interleaved gate/up rows when asked) and
// stores bf16.  No TMA tensor maps, no multicast.  Every wait is bounded; a wait that runs out raises a flag in global
// memory and all roles fall through to the common exit, where TMEM is released.
#include "skinny_gemm.cuh"

#include <atomic>

namespace mcl {

namespace {

constexpr int kTileN = 128;        // weight rows per CTA (MMA M)
constexpr int kStages = 4;
constexpr int kProducerThreads = 256;
constexpr int kThreads = kProducerThreads + 32;
constexpr int kRowBytes = 128;     // shared-memory bytes per tile row (one swizzle atom row)
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ int g_skinny_error;     // set when a bounded wait ran out (read back by tests)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait on a phase parity.  Returns false when the limit ran out or
// another role already gave up (abort flag in shared memory).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    g_skinny_error = 1;
    return false;
}

// K-major, 128-byte swizzle: 8-row groups are 1024 bytes apart; the leading
// offset is unused for swizzled K-major layouts (encoded as 1); version 1.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <int KIND_F8>
__device__ __forceinline__ void mma_issue(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND_F8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
    }
}

__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct SkinnyArgs {
    const void* w;          // [N,K] bf16 or e4m3
    const float* w_scale;   // [N] or null
    const void* x;          // [M,K] bf16 (modes 0,1) or e4m3 (mode 2)
    const float* x_scale;   // [M] (mode 2) or null
    uint16_t* y;            // [M,N] bf16 ([M,N/2] behind the SwiGLU epilogue)
    uint32_t M, N, K;
    uint32_t splits, kb_per_split;   // splits = cluster size along x
    uint32_t swiglu;        // rows 2j / 2j+1 are gate_j / up_j: store silu(g)*u
};

// swizzled byte offset of 16-byte chunk `cc` (0..7) of tile row `row`
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t cc) { return row * kRowBytes + ((cc ^ (row & 7u)) << 4); }

}  // namespace

// MODE: SKINNY_W_BF16 / SKINNY_W_E4M3 / SKINNY_W8A8.  NPAD: MMA N (16, 32 or 64).
template <int MODE, int NPAD>
__global__ void __launch_bounds__(kThreads, 2) skinny_gemm_kernel(const SkinnyArgs a) {
    constexpr int WBYTES = MODE == SKINNY_W_BF16 ? 2 : 1;          // bytes per weight element in global memory
    constexpr int XBYTES = MODE == SKINNY_W8A8 ? 1 : 2;
    constexpr int BK = MODE == SKINNY_W8A8 ? 128 : 64;             // K elements per stage
    constexpr int A_CPR = BK * WBYTES / 16;                        // 16-byte global chunks per weight row per stage
    constexpr int A_PER = kTileN * A_CPR / kProducerThreads;       // ... per producer thread
    constexpr int B_CHUNKS = NPAD * 8;                             // 16-byte chunks of the activation tile
    constexpr int B_PER = (B_CHUNKS + kProducerThreads - 1) / kProducerThreads;
    constexpr uint32_t A_STAGE = kTileN * kRowBytes, B_STAGE = NPAD * kRowBytes;
    constexpr uint32_t TMEM_COLS = NPAD < 32 ? 32 : NPAD;
    constexpr uint32_t IDESC = (1u << 4) | (MODE == SKINNY_W8A8 ? 0u : ((1u << 7) | (1u << 10))) |
                               ((uint32_t)(NPAD >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * kStages + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = base, sB = base + kStages * A_STAGE;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    const uint32_t accum_bar = bar0 + 8u * (2 * kStages);

    const uint32_t tile = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
    const uint32_t nkb = (a.K + BK - 1) / BK;
    const uint32_t kb0 = split * a.kb_per_split;
    const uint32_t kb1 = min(nkb, kb0 + a.kb_per_split);
    const uint32_t n0 = tile * kTileN;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), kProducerThreads); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    volatile int* abortp = &abort_flag;

    if (warp < kProducerThreads / 32) {
        // ------------------------------------------------------------------ producers
        const uint8_t* wg = reinterpret_cast<const uint8_t*>(a.w);
        const uint8_t* xg = reinterpret_cast<const uint8_t*>(a.x);
        uint4 ra[2][A_PER];
        uint4 rb[2][B_PER];
        auto load_a = [&](int slot, uint32_t kb) {
#pragma unroll
            for (int i = 0; i < A_PER; ++i) {
                const uint32_t c = tid + kProducerThreads * i, row = c / A_CPR, cc = c % A_CPR;
                const uint32_t n = n0 + row, k = kb * BK + cc * (16 / WBYTES);
                ra[slot][i] = (kb < kb1 && n < a.N && k < a.K)
                                  ? ld_stream16(wg + ((size_t)n * a.K + k) * WBYTES)
                                  : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        auto load_b = [&](int slot, uint32_t kb) {
#pragma unroll
            for (int i = 0; i < B_PER; ++i) {
                const uint32_t c = tid + kProducerThreads * i, row = c >> 3, cc = c & 7u;
                const uint32_t k = kb * BK + cc * (16 / XBYTES);
                rb[slot][i] = (kb < kb1 && c < B_CHUNKS && row < a.M && k < a.K)
                                  ? *reinterpret_cast<const uint4*>(xg + ((size_t)row * a.K + k) * XBYTES)
                                  : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        auto store_stage = [&](int slot, int s) {
#pragma unroll
            for (int i = 0; i < A_PER; ++i) {
                const uint32_t c = tid + kProducerThreads * i, row = c / A_CPR, cc = c % A_CPR;
                const uint4 v = ra[slot][i];
                if constexpr (MODE == SKINNY_W_E4M3) {
                    // 16 codes -> 16 bf16 holding value * 2^-120 (two 16-byte chunks)
                    uint4 lo, hi;
                    lo.x = e4m3x2_to_bf16x2_scaled<0x1404u>(v.x); lo.y = e4m3x2_to_bf16x2_scaled<0x3424u>(v.x);
                    lo.z = e4m3x2_to_bf16x2_scaled<0x1404u>(v.y); lo.w = e4m3x2_to_bf16x2_scaled<0x3424u>(v.y);
                    hi.x = e4m3x2_to_bf16x2_scaled<0x1404u>(v.z); hi.y = e4m3x2_to_bf16x2_scaled<0x3424u>(v.z);
                    hi.z = e4m3x2_to_bf16x2_scaled<0x1404u>(v.w); hi.w = e4m3x2_to_bf16x2_scaled<0x3424u>(v.w);
                    const uint32_t o0 = sA + s * A_STAGE + swz(row, 2 * cc), o1 = sA + s * A_STAGE + swz(row, 2 * cc + 1);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(o0), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(o1), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
                } else {
                    const uint32_t o = sA + s * A_STAGE + swz(row, cc);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(o), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                }
            }
#pragma unroll
            for (int i = 0; i < B_PER; ++i) {
                const uint32_t c = tid + kProducerThreads * i, row = c >> 3, cc = c & 7u;
                if (c < B_CHUNKS) {
                    uint4 v = rb[slot][i];
                    if constexpr (MODE == SKINNY_W_E4M3) {
                        // x * 2^64 (exact): keeps the products of the 2^-120-scaled weights
                        // well inside the fp32 normal range; undone in the epilogue.
                        const uint32_t two64 = 0x5F805F80u;
                        asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v.x) : "r"(two64));
                        asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v.y) : "r"(two64));
                        asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v.z) : "r"(two64));
                        asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v.w) : "r"(two64));
                    }
                    const uint32_t o = sB + s * B_STAGE + swz(row, cc);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(o), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(full_bar(s));
        };

        // weights do not depend on the producer kernel of x: two stages go out now
        load_a(0, kb0);
        load_a(1, kb0 + 1);
        pdl_trigger();
        pdl_wait();
        load_b(0, kb0);
        load_b(1, kb0 + 1);
        bool ok = true;
        uint32_t it = 0;
        for (uint32_t kb = kb0; kb < kb1 && ok; kb += 2) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (kb + j < kb1 && ok) {
                    const int s = it % kStages;
                    const uint32_t round = it / kStages;
                    if (round > 0) ok = mbar_wait(empty_bar(s), (round - 1) & 1u, abortp);
                    if (ok) {
                        store_stage(j, s);
                        load_a(j, kb + j + 2);
                        load_b(j, kb + j + 2);
                    }
                    ++it;
                }
            }
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t kb = kb0; kb < kb1 && ok; ++kb, ++it) {
            const int s = it % kStages;
            ok = mbar_wait(full_bar(s), (it / kStages) & 1u, abortp);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = make_desc(sA + s * A_STAGE), db = make_desc(sB + s * B_STAGE);
#pragma unroll
            for (int k = 0; k < 4; ++k)   // 4 x (K = 32 bytes) per 128-byte row
                mma_issue<MODE == SKINNY_W8A8>(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), IDESC,
                                               (kb > kb0 || k > 0) ? 1u : 0u);
            mma_commit(empty_bar(s));     // frees the stage once the MMAs have read it
        }
        if (ok) mma_commit(accum_bar);
    }

    // ---------------------------------------------------------------------- epilogue
    // (1) accumulator -> this CTA's shared memory, red[m][n_local] fp32 (the ring is free:
    //     every MMA that read it has completed once accum_bar fires)
    float* red = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));
    if (warp < 4) {
        const bool have = kb1 > kb0;
        const bool ok = have && mbar_wait(accum_bar, 0u, abortp);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c0 = 0; c0 < NPAD; c0 += 16) {
            uint32_t r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = 0u;
            if (ok) {
                const uint32_t taddr = tmem_base + ((warp * 32u) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) red[(c0 + j) * kTileN + warp * 32u + lane] = __uint_as_float(r[j]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    // (2) every CTA of the cluster has published its partial tile
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    // (3) this CTA finishes a contiguous slice of the tile: fixed rank order over the cluster
    {
        const uint32_t S = a.splits, rank = split;
        const uint32_t red_s = smem_u32(red);
        const bool failed = *abortp != 0;
        if (!a.swiglu) {
            const uint32_t total = a.M * kTileN;
            const uint32_t per = (total + S - 1) / S, lo = rank * per, hi = min(total, lo + per);
            for (uint32_t e = lo + tid; e < hi; e += kThreads) {
                const uint32_t m = e / kTileN, nl = e % kTileN, n = n0 + nl;
                float acc = 0.f;
                for (uint32_t r = 0; r < S; ++r) {
                    uint32_t ra;
                    float v;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(red_s + 4u * e), "r"(r));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
                    acc += v;
                }
                if (n < a.N && !failed) {
                    if constexpr (MODE == SKINNY_W_E4M3) acc *= 7.205759403792794e16f;   // 2^56 = 2^120 / 2^64
                    if (a.w_scale != nullptr) acc *= a.w_scale[n];
                    if (MODE == SKINNY_W8A8) acc *= a.x_scale[m];
                    a.y[(size_t)m * a.N + n] = f32_to_bf16_bits(acc);
                }
            }
        } else {
            const uint32_t half = kTileN / 2, total = a.M * half;
            const uint32_t per = (total + S - 1) / S, lo = rank * per, hi = min(total, lo + per);
            for (uint32_t e = lo + tid; e < hi; e += kThreads) {
                const uint32_t m = e / half, p = e % half, n = n0 + 2u * p;
                float gt = 0.f, up = 0.f;
                for (uint32_t r = 0; r < S; ++r) {
                    uint32_t ra;
                    float2 v;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(red_s + 4u * (m * kTileN + 2u * p)), "r"(r));
                    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(ra) : "memory");
                    gt += v.x;
                    up += v.y;
                }
                if (n + 1 < a.N && !failed) {
                    if constexpr (MODE == SKINNY_W_E4M3) { gt *= 7.205759403792794e16f; up *= 7.205759403792794e16f; }
                    if (a.w_scale != nullptr) { gt *= a.w_scale[n]; up *= a.w_scale[n + 1]; }
                    if (MODE == SKINNY_W8A8) { gt *= a.x_scale[m]; up *= a.x_scale[m]; }
                    const float gb = __uint_as_float((uint32_t)f32_to_bf16_bits(gt) << 16);
                    const float ub = __uint_as_float((uint32_t)f32_to_bf16_bits(up) << 16);
                    a.y[(size_t)m * (a.N / 2u) + (n >> 1)] = f32_to_bf16_bits(swiglu_f32(gb, ub));
                }
            }
        }
    }
    // (4) nobody leaves while a peer may still read its shared memory
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------
namespace {

struct Plan { uint32_t tiles, splits, kb_per_split; };

// Cluster size along K: the largest of 8/4/2/1 that keeps the grid within two CTAs
// per SM and leaves every CTA at least two K blocks.
Plan make_plan(uint32_t N, uint32_t K, uint32_t bk) {
    Plan p;
    p.tiles = (N + kTileN - 1) / kTileN;
    const uint32_t nkb = (K + bk - 1) / bk;
    const uint32_t room = 2u * (uint32_t)sm_count();
    uint32_t s = 8;
    while (s > 1 && (p.tiles * s > room || nkb / s < 2)) s >>= 1;
    p.splits = s;
    p.kb_per_split = (nkb + s - 1) / s;
    return p;
}

template <int MODE, int NPAD>
mc_status_t launch_one(const SkinnyArgs& a, uint32_t grid, cudaStream_t stream, bool pdl) {
    constexpr size_t smem = (size_t)kStages * (kTileN + NPAD) * kRowBytes + 1024;
    static_assert((size_t)NPAD * kTileN * 4 <= (size_t)kStages * (kTileN + NPAD) * kRowBytes, "reduce tile must fit in the ring");
    auto kern = skinny_gemm_kernel<MODE, NPAD>;
    static bool attr_done = false;
    if (!attr_done) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error("skinny_gemm: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
            return MC_E_CUDA;
        }
        attr_done = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = a.splits;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 2 : 1;
    (void)cudaLaunchKernelEx(&cfg, kern, a);
    MCL_CHECK_LAUNCH("skinny_gemm");
    return MC_OK;
}

template <int MODE>
mc_status_t launch_mode(const SkinnyArgs& a, uint32_t grid, cudaStream_t stream, bool pdl) {
    if (a.M <= 16) return launch_one<MODE, 16>(a, grid, stream, pdl);
    if (a.M <= 32) return launch_one<MODE, 32>(a, grid, stream, pdl);
    return launch_one<MODE, 64>(a, grid, stream, pdl);
}

}  // namespace

bool skinny_shape_ok(uint32_t N, uint32_t K, int wb) {
    return N > 0 && K > 0 && (K % (wb == 2 ? 8u : 16u)) == 0;
}

// Split-K partials travel through distributed shared memory: no global workspace.
size_t skinny_workspace_bytes(uint32_t, uint32_t, uint32_t) { return 0; }

mc_status_t skinny_gemm(int mode, const void* w, const float* w_scale, const uint16_t* x, const float* x_scale,
                        uint16_t* y, uint32_t M, uint32_t N, uint32_t K, bool swiglu, cudaStream_t stream, bool pdl) {
    if (M == 0 || M > 64 || !aligned16(w) || !aligned16(x) || (swiglu && (N & 1u))) {
        set_error("skinny_gemm: invalid args (M=%u N=%u K=%u)", M, N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    const Plan p = make_plan(N, K, mode == SKINNY_W8A8 ? 128u : 64u);
    SkinnyArgs a{};
    a.w = w; a.w_scale = w_scale; a.x = x; a.x_scale = x_scale; a.y = y;
    a.M = M; a.N = N; a.K = K; a.splits = p.splits; a.kb_per_split = p.kb_per_split; a.swiglu = swiglu ? 1u : 0u;
    const uint32_t grid = p.tiles * p.splits;
    if (mode == SKINNY_W_BF16) return launch_mode<SKINNY_W_BF16>(a, grid, stream, pdl);
    if (mode == SKINNY_W_E4M3) return launch_mode<SKINNY_W_E4M3>(a, grid, stream, pdl);
    return launch_mode<SKINNY_W8A8>(a, grid, stream, pdl);
}

// 1 when a bounded wait of the tensor-core kernel ran out since the last call (and clears it).
int skinny_take_error() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_skinny_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        const int zero = 0;
        (void)cudaMemcpyToSymbol(g_skinny_error, &zero, sizeof(int));
    }
    return v;
}

}  // namespace mcl
