// common.cuh -- shared device/host helpers of the sm_100a decode linear-layer library.
#pragma once

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>

#include <cuda_runtime.h>

#include "mc_sm100a_linear.h"

namespace mcl {

// ---- thread-local diagnostics (role of native/runtime/error.cpp:14-41) ----
void set_error(const char* fmt, ...);
void clear_error();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0u; }

// Number of SMs of the current device, cached per device id (no allocation,
// no synchronisation; cudaDeviceGetAttribute is a host-side query).
int sm_count();

// Dynamic shared memory above 48 KB has to be opted into per kernel AND per device
// (cudaFuncSetAttribute acts on the current device).  One SmemOptIn per kernel instantiation
// remembers what each device was raised to; host threads may race through it.
constexpr int kMaxDevices = 64;
struct SmemOptIn {
    std::atomic<uint32_t> set[kMaxDevices];
    std::mutex mu;
    // true when `bytes` of dynamic shared memory are usable by `kern` on the current device
    template <typename Kern>
    cudaError_t ensure(Kern kern, size_t bytes) {
        if (bytes <= 48u * 1024u) return cudaSuccess;
        int dev = 0;
        const cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        return ensure_on(dev, bytes, [&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes); });
    }
    // the bookkeeping alone: `raise` performs the opt-in on device `dev` (a fake in the host-side self-test)
    template <typename Raise>
    cudaError_t ensure_on(int dev, size_t bytes, Raise raise) {
        if (bytes <= 48u * 1024u) return cudaSuccess;
        if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
        if (set[dev].load(std::memory_order_acquire) >= bytes) return cudaSuccess;
        std::lock_guard<std::mutex> lock(mu);
        if (set[dev].load(std::memory_order_relaxed) >= bytes) return cudaSuccess;
        const cudaError_t e = raise();
        if (e == cudaSuccess) set[dev].store((uint32_t)bytes, std::memory_order_release);
        return e;
    }
    uint32_t recorded(int dev) const { return dev >= 0 && dev < kMaxDevices ? set[dev].load(std::memory_order_relaxed) : 0u; }
};

// ---- L2 prefetch of the NEXT linear's weights ------------------------------------
// A decode step is a chain of dependent kernels, and a kernel can only have as many
// weight bytes in flight before griddepcontrol.wait as its registers hold.  What hides
// the rest of the dependent-launch latency is the 126 MB L2: while kernel i computes,
// its CTAs ask the memory system (no registers, no completion to wait for) to bring the
// weights of kernel i+1 from HBM into L2, so that HBM keeps streaming through the
// bubbles between kernels and kernel i+1 reads from L2.  The caller names those weights
// with mc_sm100_hint_next_weights(); the hint applies to the next streaming launch made
// by the same host thread and is consumed by it.
struct NextWeights {
    const void* ptr;       // first byte to prefetch (16-byte aligned), nullptr = none
    uint64_t bytes;        // multiple of 16
};
NextWeights take_next_weights();     // returns the pending hint of this thread and clears it

// How the prefetch is issued (process-wide; a benchmark hook can change it):
// mode 0 = off, 1 = cp.async.bulk.prefetch.L2 in chunks of `chunk` bytes per thread, 2 = one
// prefetch.global.L2 per 128-byte line.  evict_first != 0: the demand loads of the streaming
// kernels mark their lines evict-first in L2, so that lines already consumed leave before
// lines prefetched for the next kernel.  cap = most bytes one hint may cover.
struct PrefetchConfig { uint32_t mode, chunk, evict_first; uint64_t cap; };
PrefetchConfig prefetch_config();

// Device word that bounded waits of launches made by this host thread also raise when they run
// out (besides their own flags); nullptr = none.  The decode stack points it at its failure word
// for the duration of a step, so that one status read after the step covers every kernel.
void set_wait_status_sink(int32_t* d_status);
int32_t* wait_status_sink();

// Kernel-side form: [ptr, ptr + bytes) cut into `per_cta` byte slices, one per CTA.
struct PrefetchArgs {
    const uint8_t* ptr;
    uint64_t bytes;
    uint32_t per_cta;      // multiple of 128
    uint32_t chunk;        // bytes per bulk prefetch instruction, multiple of 128 (mode 1)
    uint32_t mode;         // 0 off, 1 bulk, 2 per line
    uint32_t evict_first;  // demand loads carry the evict-first policy
};
inline PrefetchArgs make_prefetch_args(const NextWeights& nw, uint32_t ctas) {
    PrefetchArgs p{};
    const PrefetchConfig c = prefetch_config();
    p.evict_first = c.evict_first;
    if (nw.ptr == nullptr || nw.bytes == 0 || c.mode == 0 || ctas == 0) return p;
    uint64_t bytes = nw.bytes < c.cap ? nw.bytes : c.cap;
    bytes &= ~(uint64_t)15u;
    const uint64_t per = (((bytes + ctas - 1) / ctas) + 127u) & ~(uint64_t)127u;
    if (per == 0 || per > 0xFFFFFF80ull) return p;
    p.ptr = static_cast<const uint8_t*>(nw.ptr); p.bytes = bytes; p.per_cta = (uint32_t)per;
    p.chunk = c.chunk; p.mode = c.mode;
    return p;
}

// Launch with or without the programmatic-dependent-launch attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

#define MCL_CHECK_LAUNCH(what)                                                   \
    do {                                                                         \
        const cudaError_t e__ = cudaGetLastError();                              \
        if (e__ != cudaSuccess) {                                                \
            mcl::set_error("%s launch failed: %s", what, cudaGetErrorString(e__)); \
            return MC_E_CUDA;                                                    \
        }                                                                        \
    } while (0)

// ---- exchange of N-sharded outputs between the GPUs of one node ----------------
// A sharded linear stores each output element straight into EVERY rank's gathered vector
// (peer-mapped addresses) as one 32-bit word: bf16 bits in the low half, the low 16 bits of
// the exchange's sequence number in the high half.  A 32-bit store is atomic, so the word
// carries its own "valid" mark: the consumer polls the words it needs until every tag is the
// expected one -- no flag, no fence, no atomic on the critical path; the cost of an exchange
// is one NVLink store latency.  Every slot of a vector is rewritten by every exchange, so a
// slot only ever holds the current or the previous exchange's tag.  All zero = not sharded.
struct ShardIO {
    const uint32_t* step;       // device word, >= 1: index of the running step
    int32_t* status;            // set to 1 when a wait ran out (sticky: later waits give up at once)
    uint64_t timeout_ns;
    uint64_t out_peer[8];       // rank p's gathered output vector (uint32 words) as mapped here ([rank] = own)
    uint32_t world, rank;
    uint32_t in_tagged;         // 1: the activation (PRO_NONE) / the addend (PRO_RESNORM) is a tagged gathered vector
    uint32_t in_seq_mul, in_seq_add;     // its sequence number = (*step - 1) * in_seq_mul + in_seq_add
    uint32_t out_slot;          // this rank's outputs start at word rank * out_slot; 0 = outputs stay local (bf16)
    uint32_t out_seq_mul, out_seq_add;
};

constexpr unsigned long long kShardWaitDefaultNs = 1000ull * 1000ull * 1000ull;   // 1 s

// Batched (M > 1) sharded steps: the tensor-core GEMM stores its [M, rows] result straight into column
// block `rank` of EVERY rank's [M, width] activation buffer (peer-mapped) as TAGGED 64-bit words: two
// adjacent bf16 in the low half, the exchange's 32-bit sequence number (*step - 1) * layers + lsel
// (never 0; the buffers start zeroed) in the high half.  One relaxed 8-byte store per pair and peer: no
// fence, no flag, no atomics (measured on two GPUs: the same exchange behind a system-scope fence and an
// arrival counter per CTA costs ~6 us per linear; the fence waits for the stores' round trip over NVLink).
// The consumer re-reads a word until its tag is current.  world = 0: plain bf16 store to the local y.
struct PeerOut {
    uint64_t base[8];           // rank p's [M, pitch] buffer of 64-bit words as mapped here ([rank] = own)
    const uint32_t* step;       // device word >= 1: index of the running step of this kind
    uint32_t world, pitch, col0;   // pitch and col0 in WORDS (pairs of elements)
    uint32_t layers, lsel;
};
// The consumer's side: words == nullptr: the operand is plain bf16.
struct TaggedIn {
    const uint64_t* words;      // [rows, pitch] tagged words
    const uint32_t* step;
    uint32_t pitch;             // words per row
    uint32_t layers, lsel;
    uint32_t reserved;
    uint64_t timeout_ns;
    int32_t* status;            // sticky failure word
};

// Checks a caller's exchange descriptor and fills the kernel-side form.  `outs` = output
// elements this rank produces; push = false for kernels whose output stays local.
inline mc_status_t shard_io_to_args(const char* who, const mc_sm100_shard_io_t* io, uint32_t outs, bool push, ShardIO& sh) {
    if (io == nullptr || io->struct_size != sizeof(mc_sm100_shard_io_t) || io->world < 2u || io->world > 8u ||
        io->rank >= io->world || io->d_step == nullptr || io->d_status == nullptr ||
        (io->in_tagged != 0u && io->in_seq_mul == 0u && io->in_seq_add == 0u)) {
        set_error("%s: invalid exchange descriptor", who);
        return MC_E_INVALID_ARGUMENT;
    }
    sh = ShardIO{};
    sh.step = io->d_step; sh.status = io->d_status;
    sh.timeout_ns = io->timeout_ns ? io->timeout_ns : kShardWaitDefaultNs;
    sh.in_tagged = io->in_tagged ? 1u : 0u; sh.in_seq_mul = io->in_seq_mul; sh.in_seq_add = io->in_seq_add;
    sh.world = io->world; sh.rank = io->rank;
    if (push && io->out_slot != 0) {
        if (outs > io->out_slot || (io->out_seq_mul == 0u && io->out_seq_add == 0u)) {
            set_error("%s: %u outputs do not fit a slot of %u, or no output sequence number", who, outs, io->out_slot);
            return MC_E_INVALID_ARGUMENT;
        }
        for (uint32_t p = 0; p < io->world; ++p) {
            if (io->out_peer[p] == 0 || (io->out_peer[p] & 3u) != 0) {
                set_error("%s: peer %u has no output vector", who, p);
                return MC_E_INVALID_ARGUMENT;
            }
            sh.out_peer[p] = io->out_peer[p];
        }
        sh.out_slot = io->out_slot; sh.out_seq_mul = io->out_seq_mul; sh.out_seq_add = io->out_seq_add;
    }
    return MC_OK;
}

#if defined(__CUDACC__)

// ---- programmatic dependent launch ----
// wait: block until the producer grid's memory is visible (no-op when the
// kernel was not launched with the attribute).  trigger: let the dependent
// grid start its own prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }

// ---- streaming loads: read-only path, do not keep the line in L1 ----
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// The same with an L2 eviction policy (see l2_policy_stream).
__device__ __forceinline__ uint4 ld_stream16_hint(const void* p, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(policy));
    return v;
}
// evict-first: a line read once by a streaming kernel should leave L2 before lines that were
// prefetched for the next kernel and have not been read yet.
__device__ __forceinline__ uint64_t l2_policy_stream(bool evict_first) {
    uint64_t first, normal;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(first));
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(normal));
    return evict_first ? first : normal;
}

// This CTA's slice of the next kernel's weights -> L2 (no registers held, nothing to wait for).
// Bulk form: the address is 16-byte aligned and every size a multiple of 16.
__device__ __forceinline__ void prefetch_next_weights(const PrefetchArgs& p, uint32_t cta, uint32_t tid, uint32_t nthreads) {
    if (p.mode == 0u) return;
    const uint64_t lo = (uint64_t)p.per_cta * cta;
    if (lo >= p.bytes) return;
    const uint64_t hi = lo + p.per_cta < p.bytes ? lo + p.per_cta : p.bytes;
    if (p.mode == 1u) {
        for (uint64_t o = lo + (uint64_t)tid * p.chunk; o < hi; o += (uint64_t)nthreads * p.chunk) {
            const uint32_t n = (uint32_t)(hi - o < p.chunk ? hi - o : p.chunk);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.ptr + o), "r"(n) : "memory");
        }
    } else {
        for (uint64_t o = lo + (uint64_t)tid * 128u; o < hi; o += (uint64_t)nthreads * 128u)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.ptr + o));
    }
}

// ---- bf16 helpers on raw bits ----
__device__ __forceinline__ float bf16lo(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float bf16hi(uint32_t p) { return __uint_as_float(p & 0xFFFF0000u); }

// round-to-nearest-even narrowing, NaN kept quiet (same result as
// __float2bfloat16_rn for every finite input and infinities).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// fp32 fused multiply-add taking two bf16 operands directly (sm_100 mixed
// precision form): acc = a*b + acc with the exact product, one rounding.
__device__ __forceinline__ void fma_bf16(float& acc, uint16_t a, uint16_t b) {
    asm("fma.rn.f32.bf16 %0, %1, %2, %0;" : "+f"(acc) : "h"(a), "h"(b));
}

// ---- e4m3 ----
// Two e4m3 codes (bytes `lo`/`hi` selected by the PRMT selector) -> packed
// bf16x2 holding value * 2^-120 each: the 7 magnitude bits dropped at bit 4 of
// a bf16 are exponent(4)+mantissa(3) with the exponent biased by 7 instead of
// 127.  Exact for normals and subnormals; codes 0x7F/0xFF come out as 480 like
// the reference's bit decoder.
template <uint32_t SEL>
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2_scaled(uint32_t w) {
    uint32_t t;
    asm("prmt.b32 %0, %1, 0, %2;" : "=r"(t) : "r"(w), "n"(SEL));  // bytes -> [b_hi,0,b_lo,0]
    return (t & 0x80008000u) | ((t >> 4) & 0x07F007F0u);
}
// 2^120, the factor that undoes the scaling above (applied to the finished sum).
#define MCL_E4M3_UNSCALE 1.329227995784916e36f

// Hardware conversion e4m3x2 -> f16x2 (exact), then f16 -> f32 (exact).
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint16_t pair) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(pair));
    float2 r;
    asm("{.reg .f16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi;}"
        : "=f"(r.x), "=f"(r.y)
        : "r"(h2));
    return r;
}

// byte-wise decode with the reference's bit construction
// (native/kernels/sm120/kernels.h:131-148), restated.
__device__ __forceinline__ float e4m3_to_f32(uint32_t c) {
    const uint32_t sign = (c & 0x80u) << 24;
    const uint32_t mag = c & 0x7Fu;
    // value*2^-120 as fp32 bits, then exact rescale by 2^120 (subnormals of the
    // small format are fp32 subnormals here; the product is exact).
    return __uint_as_float(sign | (mag << 20)) * MCL_E4M3_UNSCALE;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}

// silu(g)*u with the reference's formula g/(1+expf(-g)) (swiglu.cu:66-69).
__device__ __forceinline__ float swiglu_f32(float g, float u) {
    return (g / (1.0f + expf(-g))) * u;
}

// ---- sharded exchange, device side ----
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t shard_tag(const ShardIO& s, uint32_t mul, uint32_t add) {
    return ((*s.step - 1u) * mul + add) & 0xFFFFu;
}

// Eight consecutive elements (32 bytes, 16-byte aligned) of a tagged gathered vector, read
// past L1 until every word carries `tag`.  The wait is bounded: after timeout_ns, or as soon
// as an earlier wait has failed, it records the failure and returns what is there.
__device__ __forceinline__ void ld_tagged8(const uint32_t* src, uint32_t tag, const ShardIO& s, uint16_t (&bits)[8]) {
    uint64_t t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        uint32_t w[8];
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "l"(src) : "memory");
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "l"(src + 4) : "memory");
        bool ok = true;
#pragma unroll
        for (int j = 0; j < 8; ++j) { ok = ok && (w[j] >> 16) == tag; bits[j] = (uint16_t)(w[j] & 0xFFFFu); }
        if (ok) return;
        if ((spins & 31u) == 0u) {
            if (*reinterpret_cast<volatile int32_t*>(s.status) != 0) return;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > s.timeout_ns) { *reinterpret_cast<volatile int32_t*>(s.status) = 1; return; }
        }
    }
}

// One tagged word (two bf16), re-read past L1 until its tag is current.  Bounded and sticky like ld_tagged8.
__device__ __forceinline__ uint32_t ld_tagged_pair(const uint64_t* src, uint32_t tag, const TaggedIn& t) {
    uint64_t t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        uint64_t w;
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(src) : "memory");
        if ((uint32_t)(w >> 32) == tag) return (uint32_t)w;
        if ((spins & 31u) == 0u) {
            if (*reinterpret_cast<volatile int32_t*>(t.status) != 0) return (uint32_t)w;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > t.timeout_ns) { *reinterpret_cast<volatile int32_t*>(t.status) = 1; return (uint32_t)w; }
        }
    }
}

#endif  // __CUDACC__

// residual add + RMSNorm over M rows whose addend is a tagged gathered buffer (add.words != nullptr, d_add ignored);
// when d_advance is given the kernel adds 1 to that word at its end.  detag_rows: tagged words -> plain bf16
// [rows, cols] (cols even), the operand form the tensor-core GEMM's TMA loads need.  Both are defined beside
// mc_sm100_residual_rmsnorm_rows.
mc_status_t residual_rmsnorm_rows_tagged(uint16_t* d_res, const uint16_t* d_add, const uint16_t* d_norm_w, uint16_t* d_out,
                                         uint32_t rows, uint32_t n, float eps, const TaggedIn& add, uint32_t* d_advance,
                                         cudaStream_t stream, bool pdl);
mc_status_t detag_rows(const TaggedIn& in, uint16_t* d_out, uint32_t rows, uint32_t cols, cudaStream_t stream, bool pdl);

}  // namespace mcl
