// sampling.cu -- top-k / top-p / temperature sampling over bf16 logits, one GPU or vocab shards.
//
// The non-greedy tail of a decode step (native/kernels/sm120/sampling.cu:253-531; launcher :731-806):
// the k strongest logits under the total order "value descending, index ascending" are found, softmaxed
// with the temperature, cut at cumulative probability top_p, renormalised, and one of them is drawn with
// the xorshift64* generator whose state lives in device memory.  The reference finds the k strongest of
// fp32 logits with two 8-bit histogram levels and a bitonic sort of up to 512 candidates, six launches
// on one GPU.  Here the logits are the bf16 the lm_head wrote, so the two histogram levels resolve the
// whole 16-bit key: the candidate set is EXACTLY the k strongest (ties at the threshold value resolved
// towards lower indices by an ordered compaction), at most 128 entries, found by one CTA per logits row
// in three passes over the row, sorted in shared memory, and the tail runs in the same kernel.
// With the vocabulary sharded over GPUs every rank does that on its shard, pushes its (at most 128)
// sorted candidates to every rank through peer-mapped memory (plain stores + one system-scope counter
// per rank, bounded wait, sticky failure word -- the protocol of the greedy pair exchange), merges the
// world * 128 candidates with the same sort and draws with its own copy of the generator state: all
// ranks hold the same state, so all ranks draw the same token.  No multicast, no collective library.
// Arithmetic of the tail follows the reference statement by statement (sequential fp32 sums in sorted
// order), so a token drawn here is the token the reference draws from the same logits and state.
#include "common.cuh"

namespace mcl {

constexpr uint32_t kSampMaxK = 128;         // native/kernels/sm120/kernels.h:689
constexpr uint32_t kSampThreads = 1024;
constexpr uint32_t kSampMergeCap = 1024;    // 8 ranks x 128 candidates

__device__ __forceinline__ uint32_t samp_rng_next(uint64_t* st) {       // sampling.cu:276-283
    uint64_t x = *st;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    *st = x;
    return (uint32_t)((x * 2685821657736338717ull) >> 32);
}

// monotonic 16-bit key of a bf16 value (sign-flip trick of sampling.cu:286-289 on the upper half)
__device__ __forceinline__ uint32_t bf16_sort_key(uint32_t bits) {
    return (bits & 0x8000u) ? (~bits & 0xFFFFu) : (bits ^ 0x8000u);
}

__device__ __forceinline__ bool samp_stronger(float va, int32_t ia, float vb, int32_t ib) {
    return (va > vb) || (va == vb && ia < ib);
}

// shared-memory bitonic sort of `cap` (power of two) entries, strongest first; all threads of the CTA
__device__ void samp_sort(float* sv, int32_t* si, uint32_t cap) {
    for (uint32_t k = 2; k <= cap; k <<= 1) {
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            for (uint32_t i = threadIdx.x; i < cap; i += blockDim.x) {
                const uint32_t l = i ^ j;
                if (l > i) {
                    const bool up = (i & k) != 0;
                    const bool a_first = samp_stronger(sv[i], si[i], sv[l], si[l]);
                    if (a_first == up) {
                        const float tv = sv[i]; const int32_t ti = si[i];
                        sv[i] = sv[l]; si[i] = si[l];
                        sv[l] = tv; si[l] = ti;
                    }
                }
            }
            __syncthreads();
        }
    }
}

// suffix scan over a 256-bin histogram: the strongest bin b with count(bins >= b) >= k; also the count of
// the bins strictly above it.  All threads of the CTA call; results in shared memory.
__device__ void samp_threshold(const uint32_t* hist, uint32_t k, uint32_t* s_bin, uint32_t* s_above, uint32_t* cum) {
    const uint32_t t = threadIdx.x;
    if (t < 256) cum[t] = hist[t];
    __syncthreads();
    for (uint32_t off = 1; off < 256; off <<= 1) {
        uint32_t v = 0;
        if (t < 256 && t >= off) v = cum[t - off];
        __syncthreads();
        if (t < 256) cum[t] += v;
        __syncthreads();
    }
    if (t == 0) { *s_bin = 0; *s_above = 0; }
    __syncthreads();
    if (t < 256) {
        const uint32_t total = cum[255];
        const uint32_t suffix_b = total - (cum[t] - hist[t]);       // count of bins >= t
        const uint32_t suffix_above = total - cum[t];               // count of bins > t
        if (suffix_b >= k && suffix_above < k) { *s_bin = t; *s_above = suffix_above; }
        if (t == 0 && total < k) { *s_bin = 0; *s_above = total - hist[0]; }   // fewer than k elements at all: take every one
    }
    __syncthreads();
}

struct SampleShard {
    const uint64_t* cand_peers;   // [world] address of each rank's exchange region as mapped here
    const uint8_t* my_region;     // this rank's own exchange region
    uint32_t* step;               // device words: [0] exchange number (>= 1), [1] rows that finished the current one
    int32_t* status;
    unsigned long long timeout_ns;
    uint32_t rank, world, max_rows;
};
// exchange region of a rank: candidate slots [world][max_rows][128] x 8 bytes, then arrival words [world][max_rows] x u32
__host__ __device__ inline size_t samp_flags_offset(uint32_t world, uint32_t max_rows) {
    return (((size_t)world * max_rows * kSampMaxK * 8u) + 255u) & ~(size_t)255u;
}

// One CTA per logits row.
__global__ void __launch_bounds__(kSampThreads, 1)
sample_topk_topp_kernel(const uint16_t* __restrict__ logits, uint32_t vocab, uint32_t row_stride, int32_t index_base,
                        const mc_sm100_sampling_config_t* __restrict__ cfgs, uint64_t* __restrict__ rng, int32_t* __restrict__ out,
                        const SampleShard sh) {
    // histogram counters: one copy per lane (bin * 32 + lane), so that the 32 lanes of a warp never meet on an
    // address or a bank even when every logit falls into the same few bins; summed into hist[] after each pass
    __shared__ uint32_t hist32[256 * 32];
    __shared__ uint32_t hist[256], cum[256];
    __shared__ uint32_t s_bin, s_above, s_count, s_ties_before[kSampThreads / 32];
    __shared__ float sv[kSampMergeCap];
    __shared__ int32_t si[kSampMergeCap];
    __shared__ int s_ok;
    pdl_trigger();
    pdl_wait();
    const uint32_t t = threadIdx.x, row = blockIdx.x, n_rows = gridDim.x;
    const uint16_t* lr = logits + (size_t)row * row_stride;
    const mc_sm100_sampling_config_t cfg = cfgs[row];
    const uint32_t k = cfg.top_k < 1u ? 1u : (cfg.top_k > kSampMaxK ? kSampMaxK : cfg.top_k);
    // contiguous chunk per thread: ties are then met in index order
    const uint32_t per = (vocab + kSampThreads - 1) / kSampThreads;
    const uint32_t lo = min(vocab, t * per), hi = min(vocab, lo + per);

    // ---- level 1: high byte of the key ----
    const uint32_t lane = t & 31u;
    auto hist_clear = [&]() { for (uint32_t i = t; i < 256u * 32u; i += kSampThreads) hist32[i] = 0; __syncthreads(); };
    auto hist_fold = [&]() {
        __syncthreads();
        if (t < 256) { uint32_t c = 0; for (uint32_t l = 0; l < 32; ++l) c += hist32[t * 32u + ((l + t) & 31u)]; hist[t] = c; }
        __syncthreads();
    };
    hist_clear();
    for (uint32_t i = lo; i < hi; ++i) atomicAdd(&hist32[(bf16_sort_key(lr[i]) >> 8) * 32u + lane], 1u);
    hist_fold();
    samp_threshold(hist, k, &s_bin, &s_above, cum);
    const uint32_t b1 = s_bin, above1 = s_above;
    // ---- level 2: low byte among the members of bin b1 ----
    hist_clear();
    for (uint32_t i = lo; i < hi; ++i) {
        const uint32_t key = bf16_sort_key(lr[i]);
        if ((key >> 8) == b1) atomicAdd(&hist32[(key & 0xFFu) * 32u + lane], 1u);
    }
    hist_fold();
    samp_threshold(hist, k - above1, &s_bin, &s_above, cum);
    const uint32_t thr = (b1 << 8) | s_bin;                      // the k-th strongest key
    const uint32_t n_gt = above1 + s_above;                      // elements strictly stronger than thr (< k)
    const uint32_t need_ties = k - n_gt;                         // of the elements equal to thr: the lowest indices
    // ---- compaction: stronger elements in any order (the sort fixes it), ties in index order ----
    if (t == 0) s_count = 0;
    for (uint32_t i = t; i < kSampMergeCap; i += kSampThreads) { sv[i] = -INFINITY; si[i] = INT32_MAX; }
    __syncthreads();
    uint32_t my_ties = 0;
    for (uint32_t i = lo; i < hi; ++i) {
        const uint32_t bits = lr[i], key = bf16_sort_key(bits);
        if (key > thr) {
            const uint32_t slot = atomicAdd(&s_count, 1u);
            sv[slot] = __uint_as_float(bits << 16);
            si[slot] = (int32_t)i + index_base;
        } else if (key == thr) {
            ++my_ties;
        }
    }
    // exclusive scan of the tie counts over the threads (warp shuffle + one pass over the warp totals)
    uint32_t incl = my_ties;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
        if ((t & 31u) >= (uint32_t)d) incl += v;
    }
    if ((t & 31u) == 31u) s_ties_before[t >> 5] = incl;
    __syncthreads();
    if (t == 0) {
        uint32_t run = 0;
        for (uint32_t w = 0; w < kSampThreads / 32; ++w) { const uint32_t c = s_ties_before[w]; s_ties_before[w] = run; run += c; }
    }
    __syncthreads();
    uint32_t tie_rank = s_ties_before[t >> 5] + incl - my_ties;   // ties before this thread's chunk
    if (my_ties != 0 && tie_rank < need_ties) {
        for (uint32_t i = lo; i < hi && tie_rank < need_ties; ++i) {
            const uint32_t bits = lr[i];
            if (bf16_sort_key(bits) == thr) {
                sv[n_gt + tie_rank] = __uint_as_float(bits << 16);
                si[n_gt + tie_rank] = (int32_t)i + index_base;
                ++tie_rank;
            }
        }
    }
    __syncthreads();
    uint32_t have = min(k, vocab);                                // candidates of this shard
    samp_sort(sv, si, kSampMaxK);

    // ---- vocab shards: every rank's sorted candidates to every rank, then merge ----
    if (sh.world > 1u) {
        const uint32_t s = *sh.step;                              // read by every row's CTA before any of them can advance it
        const size_t foff = samp_flags_offset(sh.world, sh.max_rows);
        if (t == 0) s_ok = 1;
        for (uint32_t i = t; i < sh.world * kSampMaxK; i += kSampThreads) {
            const uint32_t p = i / kSampMaxK, c = i - p * kSampMaxK;
            const uint64_t packed = (uint64_t)__float_as_uint(sv[c]) | ((uint64_t)(uint32_t)si[c] << 32);
            *reinterpret_cast<volatile uint64_t*>(reinterpret_cast<uint64_t*>(sh.cand_peers[p]) + ((size_t)sh.rank * sh.max_rows + row) * kSampMaxK + c) = packed;
        }
        __threadfence_system();
        __syncthreads();
        if (t < sh.world) {
            // "rank `rank`'s candidates of row `row` for exchange s have landed", at every rank (the word only grows)
            const uint64_t f = sh.cand_peers[t] + foff + 4ull * ((size_t)sh.rank * sh.max_rows + row);
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(s) : "memory");
            const uint32_t* mine = reinterpret_cast<const uint32_t*>(sh.my_region + foff) + (size_t)t * sh.max_rows + row;
            unsigned long long t0 = 0;
            bool ok = *reinterpret_cast<volatile int32_t*>(sh.status) == 0;
            for (uint32_t spin = 0; ok; ++spin) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
                if ((int32_t)(v - s) >= 0) break;
                if ((spin & 31u) == 31u) {
                    if (*reinterpret_cast<volatile int32_t*>(sh.status) != 0) { ok = false; break; }
                    const unsigned long long now = global_timer_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > sh.timeout_ns) { *reinterpret_cast<volatile int32_t*>(sh.status) = 1; ok = false; }
                }
            }
            if (!ok) s_ok = 0;
        }
        __syncthreads();
        const uint64_t* my_cands = reinterpret_cast<const uint64_t*>(sh.my_region);
        for (uint32_t i = t; i < kSampMergeCap; i += kSampThreads) {
            float v = -INFINITY;
            int32_t ix = INT32_MAX;
            if (s_ok && i < sh.world * kSampMaxK) {
                const uint32_t p = i / kSampMaxK, c = i - p * kSampMaxK;
                const uint64_t got = *reinterpret_cast<const volatile uint64_t*>(my_cands + ((size_t)p * sh.max_rows + row) * kSampMaxK + c);
                v = __uint_as_float((uint32_t)got);
                ix = (int32_t)(uint32_t)(got >> 32);
            }
            sv[i] = v; si[i] = ix;
        }
        __syncthreads();
        samp_sort(sv, si, kSampMergeCap);
        if (t == 0) {
            uint32_t total = 0;                                   // real candidates among the first k of the merged list
            for (uint32_t i = 0; i < k; ++i) total += si[i] != INT32_MAX ? 1u : 0u;
            have = s_ok ? total : 0u;
            // the row that finishes last advances the exchange number (every row read it before arriving here)
            __threadfence();
            if (atomicAdd(sh.step + 1, 1u) == n_rows - 1u) { sh.step[1] = 0u; __threadfence(); sh.step[0] = s + 1u; }
        }
    }

    // ---- tail (one thread; statement for statement sampling.cu:489-531) ----
    if (t != 0) return;
    if (have == 0) { out[row] = -1; return; }
    const uint32_t hsize = min(k, have);
    const float temp = cfg.temperature;
    if (!(temp > 0.f) || hsize == 1u) { out[row] = si[0]; return; }      // greedy: the generator is not consumed
    const float mx = sv[0];
    float sum = 0.f;
    for (uint32_t i = 0; i < hsize; ++i) { sv[i] = expf((sv[i] - mx) / temp); sum += sv[i]; }
    for (uint32_t i = 0; i < hsize; ++i) sv[i] /= sum;
    const float p = cfg.top_p;
    uint32_t cut = hsize;
    if (p < 1.0f) {
        float cumulative = 0.f;
        for (uint32_t i = 0; i < hsize; ++i) {
            cumulative += sv[i];
            if (cumulative >= p) { cut = i + 1; break; }
        }
    }
    float kept = 0.f;
    for (uint32_t i = 0; i < cut; ++i) kept += sv[i];
    const uint32_t r = samp_rng_next(&rng[row]);
    const float u = (float)(r >> 8) * (1.0f / 16777216.0f);
    float acc = 0.f;
    uint32_t pick = cut - 1;
    for (uint32_t i = 0; i < cut; ++i) {
        acc += sv[i] / kept;
        if (u < acc) { pick = i; break; }
    }
    out[row] = si[pick];
}

}  // namespace mcl

using namespace mcl;

extern "C" {

size_t mc_sm100_sampling_exchange_bytes(uint32_t max_rows, uint32_t world) {
    const uint32_t w = world ? world : 1u, r = max_rows ? max_rows : 1u;
    return samp_flags_offset(w, r) + (((size_t)w * r * 4u + 255u) & ~(size_t)255u);
}

static mc_status_t sample_impl(const char* who, const uint16_t* d_logits, uint32_t n_rows, uint32_t vocab, uint32_t row_stride,
                               int32_t index_base, const mc_sm100_sampling_config_t* d_cfg, uint64_t* d_rng_state,
                               int32_t* d_out_token, const SampleShard& sh, void* stream, int32_t pdl) {
    if (d_logits == nullptr || d_cfg == nullptr || d_rng_state == nullptr || d_out_token == nullptr || n_rows == 0 || n_rows > 64u ||
        vocab == 0 || row_stride < vocab) {
        set_error("%s: invalid args (rows=%u vocab=%u stride=%u)", who, n_rows, vocab, row_stride);
        return MC_E_INVALID_ARGUMENT;
    }
    (void)launch(sample_topk_topp_kernel, dim3(n_rows), dim3(kSampThreads), 0, (cudaStream_t)stream, pdl != 0, d_logits, vocab, row_stride,
                 index_base, d_cfg, d_rng_state, d_out_token, sh);
    MCL_CHECK_LAUNCH("sample_topk_topp");
    return MC_OK;
}

mc_status_t mc_sm100_sample_topk_topp(const uint16_t* d_logits, uint32_t n_rows, uint32_t vocab, uint32_t row_stride,
                                      const mc_sm100_sampling_config_t* d_cfg, uint64_t* d_rng_state, int32_t* d_out_token,
                                      void* stream, int32_t pdl) {
    clear_error();
    SampleShard sh{};
    sh.world = 1;
    return sample_impl("mc_sm100_sample_topk_topp", d_logits, n_rows, vocab, row_stride, 0, d_cfg, d_rng_state, d_out_token, sh, stream, pdl);
}

mc_status_t mc_sm100_sample_topk_topp_sharded(const uint16_t* d_logits, uint32_t n_rows, uint32_t vocab, uint32_t row_stride,
                                              int32_t index_base, const mc_sm100_sampling_config_t* d_cfg, uint64_t* d_rng_state,
                                              int32_t* d_out_token, const uint64_t* d_region_peers, const void* d_my_region,
                                              uint32_t max_rows, uint32_t* d_step, uint32_t rank, uint32_t world, uint64_t timeout_ns,
                                              int32_t* d_status, void* stream, int32_t pdl) {
    clear_error();
    if (d_region_peers == nullptr || d_my_region == nullptr || d_step == nullptr || d_status == nullptr || world < 2u || world > 8u ||
        rank >= world || max_rows == 0 || n_rows > max_rows) {
        set_error("mc_sm100_sample_topk_topp_sharded: invalid exchange args (rank=%u world=%u rows=%u max_rows=%u)", rank, world, n_rows, max_rows);
        return MC_E_INVALID_ARGUMENT;
    }
    SampleShard sh{};
    sh.cand_peers = d_region_peers; sh.my_region = static_cast<const uint8_t*>(d_my_region); sh.max_rows = max_rows;
    sh.step = d_step; sh.status = d_status; sh.timeout_ns = timeout_ns ? timeout_ns : kShardWaitDefaultNs; sh.rank = rank; sh.world = world;
    return sample_impl("mc_sm100_sample_topk_topp_sharded", d_logits, n_rows, vocab, row_stride, index_base, d_cfg, d_rng_state, d_out_token,
                       sh, stream, pdl);
}

}  // extern "C"
