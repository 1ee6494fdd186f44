// skinny_gemm.cu -- batched-decode GEMM for 4 < M <= 64 on the 5th-generation tensor cores.
//
// Y[M,N] = X[M,K] . W[N,K]^T is computed "swapped": the weight tile is the MMA's A
// operand (128 rows of W = the MMA M dimension), the activation rows are the B
// operand (MMA N = M padded to 16/32/64), so one tcgen05.mma covers 128 output
// features for every batch row and the accumulator D[128 x Mpad] (fp32) lives in
// 16..64 TMEM columns.  The kernel is still bandwidth-bound (W is streamed once);
// the tensor core only removes the per-row FMA cost that caps the CUDA-core family.
//
// Two CTAs per SM, one (row tile, K slice) work item per CTA.
//   warp 0   : TMA producer.  2-D tiled cp.async.bulk.tensor loads (no multicast) of
//              the W tile [128 x BK] and the X tile [Mpad x BK] into a ring of
//              128-byte-swizzled stages, completion on mbarriers.  The W loads of
//              the first ring-full go out before griddepcontrol.wait.
//   warp 1   : MMA issuer (one elected lane): tcgen05.mma per 32-byte K step,
//              tcgen05.commit hands each stage back to the producer.
//   warps 2-9: e4m3 weight-only form only: read the raw e4m3 tile that TMA landed,
//              widen it to bf16 (exact) into the operand ring; idle otherwise.
//   warps 2-5: epilogue: tcgen05.ld the accumulator into shared memory.
// Small N is split along K over a thread-block cluster (up to 8 CTAs per row tile):
// after a cluster barrier every CTA sums its slice of the tile over the cluster's
// partial accumulators through distributed shared memory in rank order (no atomics,
// no global scratch, bit-reproducible), applies the scales (and the SwiGLU over
// interleaved gate/up rows when asked) and stores bf16.
// Every wait is bounded; a wait that runs out raises a flag in global memory and all
// roles fall through to the common exit, where TMEM is released.
#include "skinny_gemm.cuh"

#include <cuda.h>

#include <mutex>
#include <unordered_map>

namespace mcl {

namespace {

constexpr int kTileN = 128;        // weight rows per CTA (MMA M)
constexpr int kThreads = 320;      // 10 warps
constexpr int kConvThreads = 256;  // warps 2..9
constexpr uint32_t kConvGroup = 128;  // converter threads that share one K block (two groups; four groups of 64 ran into bounded-wait timeouts and are not used)
constexpr int kRowBytes = 128;     // bytes per operand-tile row in shared memory (one swizzle row)
constexpr unsigned long long kWaitLimitNs = 200ull * 1000ull * 1000ull;   // a wait gives up after 200 ms

__device__ int g_skinny_error;     // set when a bounded wait ran out (read back by tests)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait on a phase parity.  Returns false when the limit ran out or
// another role already gave up (abort flag in shared memory).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
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
        if ((spin & 63u) == 63u) {            // look at the clock now and then; bound the wait in TIME
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) break;
        }
    }
    *abort_flag = 1;
    g_skinny_error = 1;
    if (status != nullptr) *reinterpret_cast<volatile int32_t*>(status) = 1;
    return false;
}

// 2-D tiled TMA load global -> this CTA's shared memory; x is the innermost
// (K) coordinate in elements, y the row.  x * element size is a multiple of 16 bytes
// at every call site (K steps of 64 bf16 / 64 or 128 e4m3).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
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
    const float* w_scale;   // [N] or null
    const float* x_scale;   // [M] (W8A8) or null
    uint16_t* y;            // [M,N] bf16 ([M,N/2] behind the SwiGLU epilogue)
    uint32_t M, N, K;
    uint32_t splits;        // cluster size along x = K slices per row tile
    uint32_t swiglu;        // rows 2j / 2j+1 are gate_j / up_j: store silu(g)*u
    uint32_t op_stages, raw_stages;  // ring depths (<= 8), chosen by the launcher from the grid size
    int32_t* status;        // optional device word set to 1 when a bounded wait ran out (the caller's failure word)
    PeerOut out;            // sharded step: the result goes to every rank's activation buffer as tagged words (world = 0: to y)
    PrefetchArgs pf;        // L2 prefetch of the next kernel's weights (all zero = off)
};

// swizzled byte offset of 16-byte chunk `cc` (0..7) of tile row `row`
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t cc) { return row * kRowBytes + ((cc ^ (row & 7u)) << 4); }

// Stage geometry per mode; the ring depth is a launch parameter (as many stages as fit in
// half an SM's shared memory).
template <int MODE, int NPAD> struct Ring {
    static constexpr int BK = MODE == SKINNY_W8A8 ? 128 : 64;                    // K elements per stage
    static constexpr uint32_t A_OP = kTileN * kRowBytes;                         // operand A stage (16 KB)
    static constexpr uint32_t B_OP = NPAD * kRowBytes;                           // operand B stage
    static constexpr uint32_t A_RAW = MODE == SKINNY_W_E4M3 ? kTileN * 64 : 0;   // raw e4m3 stage (8 KB)
    __host__ __device__ static constexpr uint32_t bytes(uint32_t ops, uint32_t raws) { return ops * (A_OP + B_OP) + raws * A_RAW; }
};

}  // namespace

// MODE: SKINNY_W_BF16 / SKINNY_W_E4M3 / SKINNY_W8A8.  NPAD: MMA N (16, 32 or 64).
template <int MODE, int NPAD>
__global__ void __launch_bounds__(kThreads, 2)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const SkinnyArgs a) {
    using G = Ring<MODE, NPAD>;
    constexpr int BK = G::BK;
    const uint32_t OPS = a.op_stages, RAWS = a.raw_stages;
    constexpr uint32_t TMEM_COLS = NPAD < 32 ? 32 : NPAD;
    constexpr uint32_t IDESC = (1u << 4) | (MODE == SKINNY_W8A8 ? 0u : ((1u << 7) | (1u << 10))) |
                               ((uint32_t)(NPAD >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
    constexpr bool E4 = MODE == SKINNY_W_E4M3;

    extern __shared__ uint8_t smem_raw[];
    // barriers: op_full[6] (TMA bytes landed: A+B, or B only for e4m3), op_empty[6] (MMA done with the
    // stage), conv_done[6] (e4m3: operand A written), raw_full[6], raw_empty[6], accum
    __shared__ __align__(8) uint64_t bars[41];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = base, sB = base + OPS * G::A_OP, sRaw = sB + OPS * G::B_OP;
    const uint32_t bar0 = smem_u32(bars);
    auto op_full = [&](uint32_t s) { return bar0 + 8u * s; };
    auto op_empty = [&](uint32_t s) { return bar0 + 8u * (8 + s); };
    auto conv_done = [&](uint32_t s) { return bar0 + 8u * (16 + s); };
    auto raw_full = [&](uint32_t s) { return bar0 + 8u * (24 + s); };
    auto raw_empty = [&](uint32_t s) { return bar0 + 8u * (32 + s); };
    const uint32_t accum_bar = bar0 + 8u * 40;

    const uint32_t tile = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
    const uint32_t nkb = (a.K + BK - 1) / BK;
    const uint32_t kb0 = split * nkb / a.splits, kb1 = (split + 1u) * nkb / a.splits;   // slices differ by at most one block
    const uint32_t nloc = kb1 - kb0;
    const int32_t n0 = (int32_t)(tile * kTileN);

    // the successor kernel of a chain may become resident from here on (its own first loads overlap this kernel)
    pdl_trigger();
    // W ring: operand ring (bf16 / W8A8) or raw ring (e4m3).  X always lands in the operand ring.
    const uint32_t WS = E4 ? RAWS : OPS;
    constexpr uint32_t W_BYTES = E4 ? G::A_RAW : G::A_OP;
    const uint32_t pre = nloc < WS ? nloc : WS;
    if (tid == 0) {
        abort_flag = 0;
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        for (uint32_t s = 0; s < OPS; ++s) { mbar_init(op_full(s), 1); mbar_init(op_empty(s), 1); }
        if (E4) {
            for (uint32_t s = 0; s < OPS; ++s) mbar_init(conv_done(s), kConvGroup);
            for (uint32_t s = 0; s < RAWS; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), kConvGroup); }
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // weights depend neither on the kernel that produces x nor on anything the other warps set up:
        // the first ring-full is asked for before the tensor memory and the cluster are ready
        for (uint32_t it = 0; it < pre; ++it) {
            const uint32_t bar = E4 ? raw_full(it) : op_full(it);
            mbar_expect_tx(bar, W_BYTES + (E4 ? 0u : G::B_OP));
            tma_load_2d((E4 ? sRaw : sA) + it * W_BYTES, &map_w, bar, (int32_t)((kb0 + it) * BK), n0);
        }
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // every CTA of the cluster must be running before anyone addresses a peer's shared memory: arrive now,
    // wait only in front of the epilogue's pushes (by then the barrier has long completed)
    asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    volatile int* abortp = &abort_flag;
    // warps 2..9 have nothing to do yet: they ask for the next kernel's weights (HBM -> L2)
    if (tid >= 64u) prefetch_next_weights(a.pf, blockIdx.x, tid - 64u, kThreads - 64u);

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------------------ TMA producer
            pdl_wait();
            bool ok = true;
            uint32_t itx = 0;   // next X stage to issue
            auto issue_x = [&](uint32_t it) {
                const uint32_t s = it % OPS;
                if (it >= OPS) ok = ok && mbar_wait(op_empty(s), ((it / OPS) - 1u) & 1u, abortp, a.status);
                if (!ok) return;
                if (E4) mbar_expect_tx(op_full(s), G::B_OP);
                tma_load_2d(sB + s * G::B_OP, &map_x, op_full(s), (int32_t)((kb0 + it) * BK), 0);
            };
            if constexpr (!E4) {
                for (; itx < pre && ok; ++itx) issue_x(itx);              // X of the prefetched stages
                for (uint32_t it = pre; it < nloc && ok; ++it) {          // steady state: W and X together
                    const uint32_t s = it % OPS;
                    ok = mbar_wait(op_empty(s), ((it / OPS) - 1u) & 1u, abortp, a.status);
                    if (!ok) break;
                    mbar_expect_tx(op_full(s), G::A_OP + G::B_OP);
                    tma_load_2d(sA + s * G::A_OP, &map_w, op_full(s), (int32_t)((kb0 + it) * BK), n0);
                    tma_load_2d(sB + s * G::B_OP, &map_x, op_full(s), (int32_t)((kb0 + it) * BK), 0);
                }
            } else {
                uint32_t itw = pre;
                while ((itw < nloc || itx < nloc) && ok) {
                    if (itx < nloc && itx < itw) { issue_x(itx); ++itx; }   // X never runs ahead of its raw W
                    if (itw < nloc && ok) {
                        const uint32_t s = itw % RAWS;
                        ok = mbar_wait(raw_empty(s), ((itw / RAWS) - 1u) & 1u, abortp, a.status);
                        if (!ok) break;
                        mbar_expect_tx(raw_full(s), G::A_RAW);
                        tma_load_2d(sRaw + s * G::A_RAW, &map_w, raw_full(s), (int32_t)((kb0 + itw) * BK), n0);
                        ++itw;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ------------------------------------------------------------ MMA issuer
            bool ok = true;
            for (uint32_t it = 0; it < nloc && ok; ++it) {
                const uint32_t s = it % OPS;
                const uint32_t par = (it / OPS) & 1u;
                ok = mbar_wait(op_full(s), par, abortp, a.status);
                if (ok && E4) ok = mbar_wait(conv_done(s), par, abortp, a.status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = make_desc(sA + s * G::A_OP), db = make_desc(sB + s * G::B_OP);
#pragma unroll
                for (int k = 0; k < 4; ++k)   // 4 x (K = 32 bytes) per 128-byte row
                    mma_issue<MODE == SKINNY_W8A8>(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), IDESC,
                                                   (it > 0 || k > 0) ? 1u : 0u);
                mma_commit(op_empty(s));      // frees the stage once the MMAs have read it
            }
            if (ok && nloc > 0) mma_commit(accum_bar);
        }
    } else if constexpr (E4) {
        // ---------------------------------------------------------------- e4m3 -> bf16 widening
        // thread -> (row, 16-byte raw chunk): a quarter warp covers 8 rows of one chunk column, which
        // makes the swizzled 16-byte stores of the operand tile bank-conflict free.
        // The eight warps work as groups of kConvGroup threads on alternate K blocks, so that several blocks are in
        // the (latency-bound) load -> place bits -> store -> fence chain at any time.
        const uint32_t ct = (tid - 64u) & (kConvGroup - 1u), group = (tid - 64u) / kConvGroup;
        bool ok = true;
        for (uint32_t it = group; it < nloc && ok; it += kConvThreads / kConvGroup) {
            const uint32_t sr = it % RAWS, so = it % OPS;
            ok = mbar_wait(raw_full(sr), (it / RAWS) & 1u, abortp, a.status);
            if (ok && it >= OPS) ok = mbar_wait(op_empty(so), ((it / OPS) - 1u) & 1u, abortp, a.status);
            if (!ok) break;
#pragma unroll
            for (int i = 0; i < 512 / (int)kConvGroup; ++i) {
                const uint32_t c = ct + kConvGroup * i;              // 0..511
                const uint32_t row = (c & 7u) | ((c >> 5) << 3), cc = (c >> 3) & 3u;
                uint4 v;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                             : "r"(sRaw + sr * G::A_RAW + row * 64u + cc * 16u));
                const uint32_t two120 = 0x7B807B80u;                  // 2^120 as bf16x2
                uint32_t o[8];
                o[0] = e4m3x2_to_bf16x2_scaled<0x1404u>(v.x); o[1] = e4m3x2_to_bf16x2_scaled<0x3424u>(v.x);
                o[2] = e4m3x2_to_bf16x2_scaled<0x1404u>(v.y); o[3] = e4m3x2_to_bf16x2_scaled<0x3424u>(v.y);
                o[4] = e4m3x2_to_bf16x2_scaled<0x1404u>(v.z); o[5] = e4m3x2_to_bf16x2_scaled<0x3424u>(v.z);
                o[6] = e4m3x2_to_bf16x2_scaled<0x1404u>(v.w); o[7] = e4m3x2_to_bf16x2_scaled<0x3424u>(v.w);
#pragma unroll
                for (int j = 0; j < 8; ++j) asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(o[j]) : "r"(two120));   // exact
                const uint32_t d0 = sA + so * G::A_OP + swz(row, 2 * cc), d1 = sA + so * G::A_OP + swz(row, 2 * cc + 1);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(d0), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(d1), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(conv_done(so));
            mbar_arrive(raw_empty(sr));
        }
    }

    // ---------------------------------------------------------------------- epilogue
    // The tile's 128 features are cut into S contiguous slices, one per CTA of the cluster.
    // (1) every CTA PUSHES its partial accumulator rows into the owner's shared memory
    //     (part[rank][feature][m], a region of its own behind the ring, so a push can never land
    //     in memory the owner's pipeline still uses): a thread holds 16 consecutive m of one
    //     feature after tcgen05.ld, i.e. 64 contiguous bytes = four 16-byte remote stores;
    // (2) one cluster barrier;
    // (3) each owner sums its S partials from its own shared memory in rank order, scales, stores.
    // Nothing remote is touched after the barrier, so no CTA waits for its peers before it exits.
    const uint32_t S = a.splits, rank = split;
    const uint32_t per_n = kTileN / S;                               // features per owner (S divides 128)
    constexpr uint32_t PITCH = NPAD + 4;                             // fp32 per feature row: 16-byte aligned pushes, spread banks
    const uint32_t part_s = base + G::bytes(OPS, E4 ? RAWS : 0);     // part[S][per_n][PITCH] fp32
    asm volatile("barrier.cluster.wait;" ::: "memory");              // completes the arrive of the prologue
    if (warp >= 2 && warp < 6) {
        const uint32_t q = warp & 3u;       // the TMEM lane quarter this warp may read
        const bool ok = nloc > 0 && mbar_wait(accum_bar, 0u, abortp, a.status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t nl = q * 32u + lane, owner = nl / per_n;
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote)
                     : "r"(part_s + ((rank * per_n + (nl - owner * per_n)) * PITCH) * 4u), "r"(owner));
#pragma unroll
        for (int c0 = 0; c0 < NPAD; c0 += 16) {
            uint32_t r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = 0u;
            if (ok) {
                const uint32_t taddr = tmem_base + ((q * 32u) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            }
#pragma unroll
            for (int j = 0; j < 16; j += 4)
                asm volatile("st.shared::cluster.v4.u32 [%0], {%1,%2,%3,%4};"
                             ::"r"(remote + (uint32_t)(c0 + j) * 4u), "r"(r[j]), "r"(r[j + 1]), "r"(r[j + 2]), "r"(r[j + 3]) : "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    {
        const bool failed = *abortp != 0;
        const uint32_t nbase = (uint32_t)n0 + rank * per_n;          // first feature this CTA finishes
        // sharded step: two adjacent finished values (row m, columns c and c + 1 of the result, c even) travel
        // as one tagged 64-bit word to every rank's gathered buffer
        const uint64_t out_tag = a.out.world != 0u ? (uint64_t)((*a.out.step - 1u) * a.out.layers + a.out.lsel) << 32 : 0ull;
        auto put_pair = [&](uint32_t m, uint32_t c, uint16_t v0, uint16_t v1) {
            const uint64_t word = out_tag | ((uint64_t)v1 << 16) | (uint64_t)v0;
            for (uint32_t p = 0; p < a.out.world; ++p)
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;"
                             ::"l"(reinterpret_cast<uint64_t*>(a.out.base[p]) + (size_t)m * a.out.pitch + a.out.col0 + (c >> 1)), "l"(word) : "memory");
        };
        auto partial_sum = [&](uint32_t n_rel, uint32_t m) {
            float acc = 0.f;
            for (uint32_t r = 0; r < S; ++r) {    // rank order: bit-reproducible
                float v;
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(part_s + ((r * per_n + n_rel) * PITCH + m) * 4u) : "memory");
                acc += v;
            }
            return acc;
        };
        auto finish = [&](uint32_t n_rel, uint32_t m) {       // one plain output element, scaled and rounded
            float acc = partial_sum(n_rel, m);
            const uint32_t n = nbase + n_rel;
            if (n < a.N) {
                if (a.w_scale != nullptr) acc *= a.w_scale[n];
                if (MODE == SKINNY_W8A8) acc *= a.x_scale[m];
            }
            return f32_to_bf16_bits(acc);
        };
        auto finish_swiglu = [&](uint32_t p, uint32_t m) {    // one SwiGLU output element from rows 2p, 2p + 1 of the slice
            float gt = partial_sum(2u * p, m), up = partial_sum(2u * p + 1u, m);
            const uint32_t n = nbase + 2u * p;
            if (n + 1 < a.N) {
                if (a.w_scale != nullptr) { gt *= a.w_scale[n]; up *= a.w_scale[n + 1]; }
                if (MODE == SKINNY_W8A8) { gt *= a.x_scale[m]; up *= a.x_scale[m]; }
            }
            const float gb = __uint_as_float((uint32_t)f32_to_bf16_bits(gt) << 16);
            const float ub = __uint_as_float((uint32_t)f32_to_bf16_bits(up) << 16);
            return f32_to_bf16_bits(swiglu_f32(gb, ub));
        };
        if (a.out.world != 0u) {
            // pairs of adjacent outputs (the slice holds an even number of them, starting at an even column)
            const uint32_t outs = a.swiglu ? per_n / 2u : per_n, obase = a.swiglu ? nbase >> 1 : nbase, olimit = a.swiglu ? a.N / 2u : a.N;
            for (uint32_t idx = tid; idx < (outs / 2u) * a.M; idx += kThreads) {
                const uint32_t m = idx / (outs / 2u), c_rel = 2u * (idx % (outs / 2u)), c = obase + c_rel;
                if (c < olimit && !failed) {
                    const uint16_t v0 = a.swiglu ? finish_swiglu(c_rel, m) : finish(c_rel, m);
                    const uint16_t v1 = c + 1u < olimit ? (a.swiglu ? finish_swiglu(c_rel + 1u, m) : finish(c_rel + 1u, m)) : (uint16_t)0;
                    put_pair(m, c, v0, v1);
                }
            }
        } else if (!a.swiglu) {
            for (uint32_t idx = tid; idx < per_n * a.M; idx += kThreads) {
                const uint32_t m = idx / per_n, n_rel = idx % per_n, n = nbase + n_rel;   // n fastest: coalesced stores
                float acc = partial_sum(n_rel, m);
                if (n < a.N && !failed) {
                    if (a.w_scale != nullptr) acc *= a.w_scale[n];
                    if (MODE == SKINNY_W8A8) acc *= a.x_scale[m];
                    a.y[(size_t)m * a.N + n] = f32_to_bf16_bits(acc);
                }
            }
        } else {
            for (uint32_t idx = tid; idx < (per_n / 2u) * a.M; idx += kThreads) {
                const uint32_t m = idx / (per_n / 2u), p = idx % (per_n / 2u), n = nbase + 2u * p;
                float gt = partial_sum(2u * p, m), up = partial_sum(2u * p + 1u, m);
                if (n + 1 < a.N && !failed) {
                    if (a.w_scale != nullptr) { gt *= a.w_scale[n]; up *= a.w_scale[n + 1]; }
                    if (MODE == SKINNY_W8A8) { gt *= a.x_scale[m]; up *= a.x_scale[m]; }
                    const float gb = __uint_as_float((uint32_t)f32_to_bf16_bits(gt) << 16);
                    const float ub = __uint_as_float((uint32_t)f32_to_bf16_bits(up) << 16);
                    a.y[(size_t)m * (a.N / 2u) + (n >> 1)] = f32_to_bf16_bits(swiglu_f32(gb, ub));
                }
            }
        }
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------
namespace {

struct Plan { uint32_t tiles, splits; };

// Cluster size along K: the largest of 8/4/2/1 that keeps the grid within two CTAs per SM
// and leaves every CTA at least two K blocks.
Plan make_plan(uint32_t N, uint32_t K, uint32_t bk) {
    Plan p;
    p.tiles = (N + kTileN - 1) / kTileN;
    const uint32_t nkb = (K + bk - 1) / bk;
    const uint32_t room = 2u * (uint32_t)sm_count();
    uint32_t s = 8;
    while (s > 1 && (p.tiles * s > room || nkb / s < 2)) s >>= 1;
    p.splits = s;
    return p;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Row-major [rows, K] matrix of 1- or 2-byte elements, box = [box_rows x box_k]; out-of-range
// rows / columns read as zero (ragged N, M < Mpad, K tail).
mc_status_t encode_map(CUtensorMap* map, const void* ptr, uint32_t rows, uint32_t K, uint32_t pitch, uint32_t elem_bytes,
                       uint32_t box_k, uint32_t box_rows, bool swizzle128) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) {
        set_error("skinny_gemm: cuTensorMapEncodeTiled is not available from this driver");
        return MC_E_CUDA;
    }
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch * elem_bytes};   // row pitch in bytes (a multiple of 16)
    const cuuint32_t box[2] = {box_k, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                          const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("skinny_gemm: cuTensorMapEncodeTiled failed (%d) for rows=%u K=%u", (int)r, rows, K);
        return MC_E_CUDA;
    }
    return MC_OK;
}

// An encoded tensor map depends only on (address, shape, box): a step launched eagerly would
// otherwise pay two driver encodes per GEMM.  Small process-wide cache, cleared when full.
struct MapKey {
    const void* ptr; uint32_t rows, K, pitch, elem, box_k, box_rows, swz;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && K == o.K && pitch == o.pitch && elem == o.elem && box_k == o.box_k && box_rows == o.box_rows && swz == o.swz;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = 0xCBF29CE484222325ull;
        const uint64_t v[5] = {(uint64_t)(uintptr_t)k.ptr, ((uint64_t)k.rows << 32) | k.K, ((uint64_t)k.box_k << 32) | k.box_rows,
                               ((uint64_t)k.elem << 32) | k.swz, k.pitch};
        for (uint64_t x : v) { h ^= x; h *= 0x100000001B3ull; }
        return (size_t)h;
    }
};
constexpr size_t kMapCacheMax = 4096;

mc_status_t make_map(CUtensorMap* map, const void* ptr, uint32_t rows, uint32_t K, uint32_t pitch, uint32_t elem_bytes,
                     uint32_t box_k, uint32_t box_rows, bool swizzle128) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{ptr, rows, K, pitch, elem_bytes, box_k, box_rows, swizzle128 ? 1u : 0u};
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *map = it->second; return MC_OK; }
    }
    const mc_status_t s = encode_map(map, ptr, rows, K, pitch, elem_bytes, box_k, box_rows, swizzle128);
    if (s != MC_OK) return s;
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() >= kMapCacheMax) cache.clear();
    cache.emplace(key, *map);
    return MC_OK;
}

template <int MODE, int NPAD>
mc_status_t launch_one(const void* w, const void* x, uint32_t x_pitch, const SkinnyArgs& a, uint32_t grid, cudaStream_t stream, bool pdl) {
    using G = Ring<MODE, NPAD>;
    auto kern = skinny_gemm_kernel<MODE, NPAD>;
    constexpr size_t smem_max = 112u * 1024u;
    static SmemOptIn optin;
    const cudaError_t ae = optin.ensure(kern, smem_max);
    if (ae != cudaSuccess) {
        set_error("skinny_gemm: cannot raise shared memory to %zu: %s", smem_max, cudaGetErrorString(ae));
        return MC_E_CUDA;
    }
    const size_t smem = (size_t)G::bytes(a.op_stages, MODE == SKINNY_W_E4M3 ? a.raw_stages : 0) + (size_t)(NPAD + 4) * kTileN * 4 + 2048;
    CUtensorMap map_w, map_x;
    mc_status_t s;
    if (MODE == SKINNY_W_BF16) {
        s = make_map(&map_w, w, a.N, a.K, a.K, 2, 64, kTileN, true);
        if (s == MC_OK) s = make_map(&map_x, x, a.M, a.K, x_pitch, 2, 64, NPAD, true);
    } else if (MODE == SKINNY_W_E4M3) {
        s = make_map(&map_w, w, a.N, a.K, a.K, 1, 64, kTileN, false);      // raw codes, widened by warps 2-9
        if (s == MC_OK) s = make_map(&map_x, x, a.M, a.K, x_pitch, 2, 64, NPAD, true);
    } else {
        s = make_map(&map_w, w, a.N, a.K, a.K, 1, 128, kTileN, true);
        if (s == MC_OK) s = make_map(&map_x, x, a.M, a.K, x_pitch, 1, 128, NPAD, true);
    }
    if (s != MC_OK) return s;
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
    (void)cudaLaunchKernelEx(&cfg, kern, map_w, map_x, a);
    MCL_CHECK_LAUNCH("skinny_gemm");
    return MC_OK;
}

template <int MODE>
mc_status_t launch_mode(const void* w, const void* x, uint32_t x_pitch, const SkinnyArgs& a, uint32_t grid, cudaStream_t stream, bool pdl) {
    if (a.M <= 16) return launch_one<MODE, 16>(w, x, x_pitch, a, grid, stream, pdl);
    if (a.M <= 32) return launch_one<MODE, 32>(w, x, x_pitch, a, grid, stream, pdl);
    return launch_one<MODE, 64>(w, x, x_pitch, a, grid, stream, pdl);
}

}  // namespace

// TMA needs 16-byte aligned row pitches: K % 8 (bf16 rows) and K % 16 (e4m3 rows).
bool skinny_shape_ok(uint32_t N, uint32_t K, int wb) {
    return N > 0 && K > 0 && (K % (wb == 2 ? 8u : 16u)) == 0;
}

// Split-K partials travel through distributed shared memory: no global workspace.
size_t skinny_workspace_bytes(uint32_t, uint32_t, uint32_t) { return 0; }

mc_status_t skinny_gemm(int mode, const void* w, const float* w_scale, const uint16_t* x, const float* x_scale,
                        uint16_t* y, uint32_t M, uint32_t N, uint32_t K, bool swiglu, cudaStream_t stream, bool pdl,
                        uint32_t x_pitch, const PeerOut* out) {
    if (x_pitch == 0u) x_pitch = K;
    const uint32_t x_elem = mode == SKINNY_W8A8 ? 1u : 2u;
    if (M == 0 || M > 64 || !aligned16(w) || !aligned16(x) || (swiglu && (N & 1u)) || x_pitch < K || ((x_pitch * x_elem) & 15u) != 0u) {
        set_error("skinny_gemm: invalid args (M=%u N=%u K=%u x_pitch=%u)", M, N, K, x_pitch);
        return MC_E_INVALID_ARGUMENT;
    }
    const Plan p = make_plan(N, K, mode == SKINNY_W8A8 ? 128u : 64u);
    SkinnyArgs a{};
    a.w_scale = w_scale; a.x_scale = x_scale; a.y = y;
    a.M = M; a.N = N; a.K = K; a.splits = p.splits; a.swiglu = swiglu ? 1u : 0u;
    const uint32_t grid = p.tiles * p.splits;
    a.pf = make_prefetch_args(take_next_weights(), grid);
    a.status = wait_status_sink();
    if (out != nullptr) a.out = *out;
    // Ring depth: as many stages as fit in ~108 KB, i.e. half an SM's shared memory.  Measured
    // (down_proj 2304 x 5760, chain of calls): with 150 or 200 KB, one CTA per SM, a call takes 14.7 us
    // against 8.8 us at M = 8 and 19.1 against 12.9 us at M = 64, because the next kernel's CTA can then
    // no longer become resident (and prefetch its weights) while this one drains.
    const uint32_t npad = M <= 16 ? 16u : (M <= 32 ? 32u : 64u);
    const uint32_t op_stage = (uint32_t)(kTileN + npad) * kRowBytes;
    const uint32_t budget = 108u * 1024u - (npad + 4u) * kTileN * 4u - 1024u;  // minus the split-K exchange region
    if (mode == SKINNY_W_E4M3) {
        // operand ring of 3 (2 when the raw ring would otherwise drop below 2 stages)
        a.op_stages = (budget >= 3u * op_stage + 2u * kTileN * 64u) ? 3u : 2u;
        a.raw_stages = (budget - a.op_stages * op_stage) / (kTileN * 64u);
        if (a.raw_stages > 8u) a.raw_stages = 8u;
        if (a.raw_stages < 2u) a.raw_stages = 2u;
    } else {
        a.op_stages = budget / op_stage;
        if (a.op_stages > 8u) a.op_stages = 8u;
        if (a.op_stages < 2u) a.op_stages = 2u;
        a.raw_stages = 1u;
    }
    if (mode == SKINNY_W_BF16) return launch_mode<SKINNY_W_BF16>(w, x, x_pitch, a, grid, stream, pdl);
    if (mode == SKINNY_W_E4M3) return launch_mode<SKINNY_W_E4M3>(w, x, x_pitch, a, grid, stream, pdl);
    return launch_mode<SKINNY_W8A8>(w, x, x_pitch, a, grid, stream, pdl);
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
