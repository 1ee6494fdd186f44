// decode_chain.cu -- one M = 1 decode step (every linear of every layer and the lm_head) as ONE
// persistent kernel.
//
// Why: launched one kernel per linear, the chain leaves HBM idle at every dependency: a kernel can
// hold only what fits its registers in flight before it may read its activation, and between the
// last byte of one linear and the first multiply of the next lie the grid dependency, the
// activation fetch and the prologue.  Here the weight stream never stops at a dependency:
//   * one CTA per SM (cooperative launch: all CTAs are resident), 16 warps;
//   * every linear's rows are dealt to the CTAs as contiguous ranges and a CTA's range is cut into
//     units of a few whole rows (9-12 KB: the copy engine of an SM takes ~0.2 us per request whatever
//     its size, measured, so smaller units cannot reach the HBM rate).  The units of ALL linears, in
//     chain order, are dealt round-robin to the warps; warp w owns slot w of a 16-slot shared-memory
//     ring (nearly the whole SM, ~150-185 KB);
//   * a warp waits for its slot's mbarrier, multiplies the rows against the activation in shared
//     memory (same lane -> element assignment and the same accumulation order as
//     gemv_fast_kernel: results are bit-equal to the per-linear kernels), stores, and at once asks
//     for its NEXT unit with one cp.async.bulk -- no registers, no tensor map, no multicast --
//     whichever linear that unit belongs to.  So the weights of the next linear(s) arrive while the
//     current one still waits for its activation.  (A single thread issuing the copies for all
//     slots was measured: ~0.6 us per unit, a third of the HBM rate.);
//   * a linear's output vector goes through global memory (L2) as TAGGED words (bf16 bits | 16-bit
//     sequence number), so a reader can tell a current word from a stale one without any fence.
//     When all warps of a CTA are done with a linear, one thread adds 1 to that linear's arrival
//     counter (relaxed, no fence) and polls it (one poller per CTA) until all CTAs have arrived;
//     only then do the CTA's threads read the words past L1, re-reading the rare word whose tag is
//     not current yet.  Both simpler forms were measured and are slower: every thread polling the
//     tagged words from the start (the polls of 148 x 288 threads on the same 72 lines delay the
//     very stores they wait for: 3-13 us per linear), and plain words behind a release / acquire
//     pair on the counter (each fence costs about a microsecond here: 3.5 us per linear).
//     Counters only ever grow (target = step x CTAs): nothing is reset between steps.  The
//     residual stream lives in every CTA's shared memory (each CTA needs the whole normalised
//     vector anyway);
//   * the greedy token: per-CTA best logit -> global candidates, the last CTA to arrive (one
//     atomic ticket) reduces them.
// Every wait is bounded in time.  A wait that runs out sets the failure word, every later wait
// of the step gives up at once, the kernel drains its copies and ends normally.
#include "decode_chain.cuh"

#include "gemv_fast.cuh"

namespace mcl {

namespace {

constexpr int kWarps = 16;                  // consumer warps = ring slots
constexpr int kConsumers = kWarps * 32;
constexpr int kThreads = kConsumers;
constexpr uint32_t kSmemLimit = 227u * 1024u;
constexpr uint32_t kStaticSmem = 1024u;     // barriers, reduction scratch (upper bound)

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// named barrier 1: the 512 threads of the CTA (kept apart from barrier 0, which brackets the kernel)
__device__ __forceinline__ void cbar_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ __forceinline__ bool cbar_or(bool p) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 1, 512, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)(p ? 1u : 0u))
        : "memory");
    return r != 0u;
}

struct Waiter {
    volatile int* abort_flag;   // shared: some wait of this CTA ran out
    int32_t* status;            // global failure word
    uint64_t timeout_ns;
};

__device__ __forceinline__ void give_up(const Waiter& w) {
    *w.abort_flag = 1;
    *reinterpret_cast<volatile int32_t*>(w.status) = 1;
}

// Bounded wait on an mbarrier phase; false when the step has failed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const Waiter& w) {
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if (*w.abort_flag) return false;
        if ((spin & 63u) == 0u) {
            if (*reinterpret_cast<volatile int32_t*>(w.status) != 0) { *w.abort_flag = 1; return false; }
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > w.timeout_ns) break;
        }
    }
    give_up(w);
    return false;
}

// Eight consecutive words of a tagged vector, re-read past L1 until every word carries `tag` (bounded).
__device__ __forceinline__ void poll_tagged8(const uint32_t* src, uint32_t tag, const Waiter& w, uint16_t (&bits)[8]) {
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; ++spin) {
        uint32_t v[8];
        asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(src) : "memory");
        asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "l"(src + 4) : "memory");
        bool ok = true;
#pragma unroll
        for (int j = 0; j < 8; ++j) { ok = ok && (v[j] >> 16) == tag; bits[j] = (uint16_t)(v[j] & 0xFFFFu); }
        if (ok) return;
        if (*w.abort_flag) return;
        __nanosleep(64);
        if ((spin & 31u) == 0u) {
            if (*reinterpret_cast<volatile int32_t*>(w.status) != 0) { *w.abort_flag = 1; return; }
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > w.timeout_ns) { give_up(w); return; }
        }
    }
}

__device__ __forceinline__ uint32_t chain_tag(uint32_t step, uint32_t count, uint32_t linear) {
    return ((step - 1u) * count + linear + 1u) & 0xFFFFu;
}

// This CTA's arrival at a linear's counter (one thread, after the CTA's barrier).  Relaxed: the data is
// validated by its tags, the counter only says when looking at it is worth while.
__device__ __forceinline__ void chain_arrive(uint32_t* ctr) {
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
}
// Bounded wait until every CTA has arrived (one thread).
__device__ __forceinline__ void chain_wait(const uint32_t* ctr, uint32_t target, const Waiter& w) {
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; ++spin) {
        uint32_t v;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
        if ((int32_t)(v - target) >= 0) return;
        if (*w.abort_flag) return;
        __nanosleep(20);
        if ((spin & 31u) == 0u) {
            if (*reinterpret_cast<volatile int32_t*>(w.status) != 0) { *w.abort_flag = 1; return; }
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > w.timeout_ns) { give_up(w); return; }
        }
    }
}

// One 16-byte unit's worth of activation in registers (bf16: 8 elements; e4m3: 16 elements as f16).
template <int WB> struct XUnit;
template <> struct XUnit<2> { uint4 a; };
template <> struct XUnit<1> { uint4 a, b; };
template <int WB>
__device__ __forceinline__ XUnit<WB> load_x(const uint16_t* xb, const uint16_t* xh, uint32_t v) {
    XUnit<WB> x;
    if constexpr (WB == 2) {
        x.a = reinterpret_cast<const uint4*>(xb)[v];
    } else {
        x.a = reinterpret_cast<const uint4*>(xh)[2u * v];
        x.b = reinterpret_cast<const uint4*>(xh)[2u * v + 1u];
    }
    return x;
}
// e4m3 on CUDA cores: same element -> accumulator assignment and order as mac_wide
__device__ __forceinline__ void mac_x(const WideUnit<1>& w, const XUnit<1>& x, float2& a, float2& b) {
    const uint32_t xv[8] = {x.a.x, x.a.y, x.a.z, x.a.w, x.b.x, x.b.y, x.b.z, x.b.w};
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
        fma_f16(a.x, (uint16_t)(w.h[j] & 0xFFFFu), (uint16_t)(xv[j] & 0xFFFFu));
        fma_f16(a.y, (uint16_t)(w.h[j] >> 16), (uint16_t)(xv[j] >> 16));
        fma_f16(b.x, (uint16_t)(w.h[j + 1] & 0xFFFFu), (uint16_t)(xv[j + 1] & 0xFFFFu));
        fma_f16(b.y, (uint16_t)(w.h[j + 1] >> 16), (uint16_t)(xv[j + 1] >> 16));
    }
}

__device__ __forceinline__ ChainLinear load_linear(const ChainLinear* table, uint32_t i) {
    ChainLinear lin;
    const uint4* src = reinterpret_cast<const uint4*>(table + i);
    uint4* dst = reinterpret_cast<uint4*>(&lin);
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j] = __ldg(src + j);
    return lin;
}

}  // namespace

template <int WB>
__global__ void __launch_bounds__(kThreads, 1) decode_chain_kernel(const ChainArgs a) {
    extern __shared__ __align__(128) uint8_t chain_smem[];
    __shared__ __align__(8) uint64_t bar_full[kWarps];
    __shared__ float red_f[kWarps];
    __shared__ int32_t red_i[kWarps];
    __shared__ int abort_flag, last_flag;
    __shared__ uint32_t units_done[kWarps], units_asked[kWarps];
    // this CTA's rows [lo, hi) and unit count per distinct linear shape (the 64-bit divisions are done once)
    __shared__ uint32_t sh_lo[CHAIN_SHAPES], sh_hi[CHAIN_SHAPES], sh_units[CHAIN_SHAPES];

    // dynamic shared memory: ring slots | [e4m3: x as f16, kmax] | x as bf16, kmax | residual bf16, H
    uint8_t* slots = chain_smem;
    uint16_t* xh = reinterpret_cast<uint16_t*>(slots + (size_t)kWarps * a.slot_bytes);
    uint16_t* xb = xh + (WB == 1 ? a.kmax : 0u);
    uint16_t* res_s = xb + a.kmax;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t cta = blockIdx.x, G = gridDim.x;
    if (tid >= 32u && tid < 32u + a.nshapes) {
        const uint32_t i = tid - 32u;
        const uint64_t n = a.shape_rows[i] / a.shape_gran[i];
        const uint32_t lo = a.shape_gran[i] * (uint32_t)(n * cta / G), hi = a.shape_gran[i] * (uint32_t)(n * (cta + 1u) / G);
        sh_lo[i] = lo; sh_hi[i] = hi; sh_units[i] = (hi - lo + a.shape_rpu[i] - 1u) / a.shape_rpu[i];
    }
    if (tid == 0) {
        abort_flag = 0;
        last_flag = 0;
        for (int s = 0; s < kWarps; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bar_full[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    Waiter wt;
    wt.abort_flag = &abort_flag;
    wt.status = a.status;
    wt.timeout_ns = a.timeout_ns;
    const uint32_t step = *reinterpret_cast<volatile const uint32_t*>(a.step);
    const uint32_t count = a.count;

    {
        // ------------------------------------------------------------------ the working warps
        const uint8_t* slot_p = slots + (size_t)warp * a.slot_bytes;
        const uint32_t slot = smem_addr(slot_p), bar = smem_addr(&bar_full[warp]);
        uint64_t policy;
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
        // the copy cursor: this warp's next unit to ask for is unit pj of linear pL (of this CTA's units)
        uint32_t pL = 0, pj = warp, p_lo = 0, p_units = 0, p_rpu = 1, p_row_bytes = 0, p_hi = 0, asked = 0;
        const uint8_t* p_w = nullptr;
        auto ask_next = [&]() {
            while (pL < count && pj >= p_units) {        // on to the linear that holds the unit (the first call loads linear 0)
                pj -= p_units;
                if (p_row_bytes != 0u) ++pL;
                if (pL >= count) break;
                const ChainLinear pl = load_linear(a.table, pL);
                p_lo = sh_lo[pl.shape]; p_hi = sh_hi[pl.shape]; p_units = sh_units[pl.shape];
                p_rpu = pl.rows_per_unit;
                p_row_bytes = pl.K * WB;
                p_w = pl.w;
            }
            if (pL >= count) return;
            const uint32_t row = p_lo + pj * p_rpu;
            const uint32_t bytes = (p_hi - row < p_rpu ? p_hi - row : p_rpu) * p_row_bytes;   // a multiple of 16, as is the source offset
            if (lane == 0) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                    ::"r"(slot), "l"(p_w + (size_t)row * p_row_bytes), "r"(bytes), "r"(bar), "l"(policy)
                    : "memory");
            }
            ++asked;
            pj += kWarps;
        };
        ask_next();
        // The step's small operands (the table, the norm weights, the row scales) -> L2, every warp of every
        // CTA a share: read on demand later they would queue behind the weight stream.
        for (uint32_t L = cta * kWarps + warp; L < count; L += G * kWarps) {
            const ChainLinear lin = load_linear(a.table, L);
            if (lane == 0 && L + G * kWarps < count) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.table + L + G * kWarps));
            if (lin.norm_w != nullptr)
                for (uint32_t o = lane * 128u; o < lin.K * 2u; o += 32u * 128u)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t*>(lin.norm_w) + o));
            if (lin.scale != nullptr)
                for (uint32_t o = lane * 128u; o < lin.N * 4u; o += 32u * 128u)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t*>(lin.scale) + o));
        }
        uint32_t q_base = 0, my_units = 0;
        float best_v = -INFINITY;
        int32_t best_i = INT32_MAX;
        for (uint32_t L = 0; L < count; ++L) {
            const ChainLinear lin = load_linear(a.table, L);
            const uint32_t K = lin.K, nchunk = K / 8u;
            // ---- the activation: the previous linear's output -> (prologue) -> shared memory
            // norm weights do not depend on anything this step computes: ask for them before any wait
            uint4 nw_first = make_uint4(0u, 0u, 0u, 0u);
            if (lin.pro == PRO_RESNORM && tid < nchunk) nw_first = __ldg(reinterpret_cast<const uint4*>(lin.norm_w) + tid);
            cbar_sync();            // every warp is done with the previous linear: its activation is free, its outputs are stored
            if (L > 0u) {
                if (tid == 0) {
                    chain_arrive(a.arrivals + (L - 1u));
                    chain_wait(a.arrivals + (L - 1u), step * G, wt);
                }
                cbar_sync();        // every CTA has stored its part of the previous linear's output
            }
            bool inexact = false;
            const uint32_t in_tag = lin.in_buf < CHAIN_BUFS ? chain_tag(step, count, L - 1u) : 0u;
            const uint32_t* in_words = lin.in_buf < CHAIN_BUFS ? a.bufs[lin.in_buf] : nullptr;
            if (lin.pro == PRO_NONE) {
                for (uint32_t c = tid; c < nchunk; c += kConsumers) {
                    uint16_t bits[8];
                    poll_tagged8(in_words + 8u * c, in_tag, wt, bits);
                    put_x8<WB>(xh, xb, c, bits, inexact);
                }
            } else {
                // res = bf16(res + addend); the norm reads the ROUNDED residual (rmsnorm.cu:144-154)
                float ss = 0.f;
                for (uint32_t c = tid; c < nchunk; c += kConsumers) {
                    uint16_t rb[8], ad[8];
                    unpack8(lin.in_buf == CHAIN_IN_X ? __ldg(reinterpret_cast<const uint4*>(a.x_in) + c) : reinterpret_cast<const uint4*>(res_s)[c], rb);
                    if (in_words != nullptr) poll_tagged8(in_words + 8u * c, in_tag, wt, ad);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float r = __uint_as_float((uint32_t)rb[j] << 16);
                        if (in_words != nullptr) {
                            r += __uint_as_float((uint32_t)ad[j] << 16);
                            rb[j] = f32_to_bf16_bits(r);
                            r = __uint_as_float((uint32_t)rb[j] << 16);
                        }
                        ss = fmaf(r, r, ss);
                    }
                    uint4 q4;
                    q4.x = rb[0] | ((uint32_t)rb[1] << 16); q4.y = rb[2] | ((uint32_t)rb[3] << 16);
                    q4.z = rb[4] | ((uint32_t)rb[5] << 16); q4.w = rb[6] | ((uint32_t)rb[7] << 16);
                    reinterpret_cast<uint4*>(res_s)[c] = q4;
                }
                ss = warp_sum(ss);
                if (lane == 0) red_f[warp] = ss;
                cbar_sync();
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) tot += red_f[w];   // fixed order
                const float inv = 1.0f / sqrtf(tot / (float)K + a.eps);
                for (uint32_t c = tid; c < nchunk; c += kConsumers) {   // same thread, same chunks as pass 1
                    uint16_t nw[8], rb[8], bits[8];
                    unpack8(c == tid ? nw_first : __ldg(reinterpret_cast<const uint4*>(lin.norm_w) + c), nw);
                    unpack8(reinterpret_cast<const uint4*>(res_s)[c], rb);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        bits[j] = f32_to_bf16_bits(__uint_as_float((uint32_t)rb[j] << 16) * inv * __uint_as_float((uint32_t)nw[j] << 16));
                    put_x8<WB>(xh, xb, c, bits, inexact);
                }
            }
            const bool fallback = cbar_or(inexact);     // also the staging barrier
            const bool skip_mac = (WB == 1) && fallback;

            // ---- this warp's units of the linear
            const uint32_t lo = sh_lo[lin.shape], hi = sh_hi[lin.shape], units = sh_units[lin.shape], rpu = lin.rows_per_unit;
            const uint32_t row_bytes = K * WB, nvec = row_bytes / 16u, per_lane = (nvec + 31u) / 32u;
            // K = 2304 (every linear but down_proj at the benchmark's shapes): this lane's slice of the activation
            // stays in registers for the whole linear, so that only the weights cross the shared-memory port
            constexpr int XR = WB == 2 ? 9 : 5;
            XUnit<WB> xr[XR];
            const bool x_in_regs = per_lane == (uint32_t)XR;
            if (x_in_regs) {
#pragma unroll
                for (int u = 0; u < XR; ++u) {
                    const uint32_t v = lane + 32u * (uint32_t)u;
                    xr[u] = load_x<WB>(xb, xh, v < nvec ? v : 0u);
                }
            }
            const uint32_t out_tag = chain_tag(step, count, L) << 16;
            uint32_t* out_words = lin.out_buf < CHAIN_BUFS ? a.bufs[lin.out_buf] : nullptr;
            for (uint32_t j = (warp + kWarps - (q_base & (kWarps - 1u))) & (kWarps - 1u); j < units; j += kWarps) {
                const uint32_t row0 = lo + j * rpu, nrows = hi - row0 < rpu ? hi - row0 : rpu;
                float sc_lane = 1.f;
                if constexpr (WB == 1) {
                    if (lane < nrows) sc_lane = __ldg(lin.scale + row0 + lane);
                }
                if (!mbar_wait(bar, my_units & 1u, wt)) break;
                ++my_units;
                for (uint32_t r = 0; r < nrows; r += 2u) {
                    const bool two = r + 1u < nrows;
                    // the multiply-accumulate of gemv_fast_kernel, operation for operation.  bf16 (tensor cores): rows r and
                    // r + 1 are A rows g and 8 + g, every lane takes part in every mma (zeros beyond the row's last unit or
                    // without a second row)
                    // bf16: row r in (a01, b01), row r + 1 in (a23, b23).  e4m3 (CUDA cores): row r in (a01, b01) = (acc_a, acc_b)
                    // of gemv_fast_kernel, row r + 1 in (a23, b23)
                    MmaAcc md;
                    md.a01 = md.a23 = md.b01 = md.b23 = make_float2(0.f, 0.f);
                    if (!skip_mac) {
                        const uint8_t* w0 = slot_p + (size_t)r * row_bytes;
                        const uint8_t* w1 = w0 + row_bytes;
                        auto unit = [&](uint32_t v, const XUnit<WB>& xv) {
                            const bool in = v < nvec;
                            const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
                            WideUnit<WB> wu0, wu1;
                            widen(in ? reinterpret_cast<const uint4*>(w0)[v] : z4, wu0);
                            widen(in && two ? reinterpret_cast<const uint4*>(w1)[v] : z4, wu1);
                            if constexpr (WB == 2) {
                                mac_mma(wu0, &wu1, in ? xv.a : z4, md);
                            } else if (in) {
                                mac_x(wu0, xv, md.a01, md.b01);
                                if (two) mac_x(wu1, xv, md.a23, md.b23);
                            }
                        };
                        if (x_in_regs) {
#pragma unroll
                            for (int u = 0; u < XR; ++u) unit(lane + 32u * (uint32_t)u, xr[u]);
                        } else {
#pragma unroll 3
                            for (uint32_t u = 0; u < per_lane; ++u) {
                                const uint32_t v = lane + 32u * u;
                                unit(v, load_x<WB>(xb, xh, v < nvec ? v : 0u));
                            }
                        }
                    }
                    float tot[2];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const uint32_t row = row0 + r + (uint32_t)i;
                        float s = WB == 2 ? warp_sum(mma_row(md, i, lane))
                                          : warp_sum(i == 0 ? (md.a01.x + md.a01.y) + (md.b01.x + md.b01.y) : (md.a23.x + md.a23.y) + (md.b23.x + md.b23.y));
                        if constexpr (WB == 1) {
                            s *= kF16Unscale;
                            if ((fallback || s != s) && row < hi && (i == 0 || two))   // warp-uniform: s is the same in every lane
                                s = fp8_row_exact(lin.w + (size_t)row * row_bytes, xb, nvec, lane);
                            s *= __shfl_sync(0xffffffffu, sc_lane, (int)((r + (uint32_t)i) & 31u));
                        }
                        tot[i] = s;
                    }
                    if (lin.epi == EPI_SWIGLU) {
                        if (lane == 0 && two) {
                            const float gt = __uint_as_float((uint32_t)f32_to_bf16_bits(tot[0]) << 16);
                            const float up = __uint_as_float((uint32_t)f32_to_bf16_bits(tot[1]) << 16);
                            const uint32_t yb = f32_to_bf16_bits(swiglu_f32(gt, up));
                            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(out_words + ((row0 + r) >> 1)), "r"(out_tag | yb) : "memory");
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            if (i == 1 && !two) break;
                            const uint32_t row = row0 + r + (uint32_t)i;
                            const uint16_t yb = f32_to_bf16_bits(tot[i]);
                            if (lin.epi == EPI_ARGMAX) {
                                if (lane == 0) a.logits[row] = yb;
                                const float v = __uint_as_float((uint32_t)yb << 16);
                                if (v > best_v || (v == best_v && (int32_t)row < best_i)) { best_v = v; best_i = (int32_t)row; }
                            } else if (lane == 0) {
                                asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(out_words + row), "r"(out_tag | (uint32_t)yb) : "memory");
                            }
                        }
                    }
                }
                __syncwarp();           // every lane has its weights in registers: the slot is free for the next unit
                ask_next();
            }
            q_base += units;
        }

        // ---- the greedy token: CTA best -> candidates; the last CTA to arrive reduces them
        if (lane == 0) { red_f[warp] = best_v; red_i[warp] = best_i; }
        cbar_sync();
        if (tid == 0) {
            float bv = red_f[0];
            int32_t bi = red_i[0];
            for (int w = 1; w < kWarps; ++w)
                if (red_f[w] > bv || (red_f[w] == bv && red_i[w] < bi)) { bv = red_f[w]; bi = red_i[w]; }
            a.stage_val[cta] = bv;
            a.stage_idx[cta] = bi;
            __threadfence();
            const uint32_t ticket = atomicInc(a.ticket, G - 1u);      // wraps to 0 with the last arrival
            last_flag = ticket == G - 1u ? 1 : 0;
        }
        cbar_sync();
        if (last_flag) {
            __threadfence();
            float bv = -INFINITY;
            int32_t bi = INT32_MAX;
            for (uint32_t c = tid; c < G; c += kConsumers) {
                const float v = *reinterpret_cast<volatile const float*>(a.stage_val + c);
                const int32_t i = *reinterpret_cast<volatile const int32_t*>(a.stage_idx + c);
                if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
            }
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, s);
                const int32_t oi = __shfl_xor_sync(0xffffffffu, bi, s);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            cbar_sync();            // tid 0 has read red_f / red_i above
            if (lane == 0) { red_f[warp] = bv; red_i[warp] = bi; }
            cbar_sync();
            if (tid == 0) {
                for (int w = 1; w < kWarps; ++w)
                    if (red_f[w] > bv || (red_f[w] == bv && red_i[w] < bi)) { bv = red_f[w]; bi = red_i[w]; }
                a.token[0] = bi;
                if (a.token_val != nullptr) a.token_val[0] = bv;
                *a.step = step + 1u;
            }
        }
        // a failed step: the copy this warp's slot still expects must land before the CTA may go
        if (lane == 0) { units_done[warp] = my_units; units_asked[warp] = asked; }
    }
    __syncthreads();
    if (abort_flag && warp < kWarps && lane == 0) {
        const uint32_t mine = units_asked[warp];
        if (mine > units_done[warp]) {
            Waiter drain = wt;
            int never = 0;
            drain.abort_flag = &never;
            (void)mbar_wait(smem_addr(&bar_full[warp]), (mine - 1u) & 1u, drain);
        }
    }
}

// ---- host side ---------------------------------------------------------------------------

uint32_t chain_rows_per_unit(int wb, uint32_t K, uint32_t epi, uint32_t slot_bytes) {
    const uint32_t row_bytes = K * (uint32_t)wb, gran = epi == EPI_SWIGLU ? 2u : 1u;
    uint32_t rows = slot_bytes / row_bytes;
    if (rows > 32u) rows = 32u;              // the row scales of a unit travel one per lane
    rows -= rows % gran;
    return rows;
}

size_t chain_smem_bytes(int wb, uint32_t H, uint32_t kmax, uint32_t slot_bytes) {
    return (size_t)kWarps * slot_bytes + (size_t)kmax * 2u * (wb == 1 ? 2u : 1u) + (size_t)H * 2u;
}

uint32_t chain_slot_bytes(int wb, uint32_t H, uint32_t kmax, uint32_t max_unit_bytes) {
    const size_t fixed = chain_smem_bytes(wb, H, kmax, 0) + kStaticSmem + 128u;
    if (fixed >= kSmemLimit) return 0;
    uint32_t slot = (uint32_t)((kSmemLimit - fixed) / kWarps) & ~127u;
    if (slot < max_unit_bytes) return 0;
    return slot;
}

mc_status_t decode_chain_launch(int wb, const ChainArgs& a, cudaStream_t stream) {
    const size_t smem = chain_smem_bytes(wb, a.H, a.kmax, a.slot_bytes);
    cudaError_t e;
    if (wb == 2) { static SmemOptIn optin; e = optin.ensure(decode_chain_kernel<2>, smem); }
    else { static SmemOptIn optin; e = optin.ensure(decode_chain_kernel<1>, smem); }
    if (e != cudaSuccess) {
        set_error("decode chain: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        return MC_E_CUDA;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)sm_count());
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;      // every CTA resident: the CTAs wait for one another's outputs
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (wb == 2) (void)cudaLaunchKernelEx(&cfg, decode_chain_kernel<2>, a);
    else (void)cudaLaunchKernelEx(&cfg, decode_chain_kernel<1>, a);
    MCL_CHECK_LAUNCH("decode_chain");
    return MC_OK;
}

}  // namespace mcl
