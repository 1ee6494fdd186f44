// stack.cu -- the decode linear stack as one host-side object: weight-arena layout,
// linear dispatch per step, CUDA-graph replay, host-buffer step.
//
// This is the slice of the reference's executors that belongs to the linear path:
// the per-layer dispatch of run_real_forward (native/runtime/forward.cpp:98-160,
// 206-237, 306-373, 443-462) and of mc_batch_step (native/runtime/batch_group.cpp:745-807),
// the compact 256-byte-aligned placement of the weight sections
// (native/runtime/weight_loader.cpp:355-365, 563-630) and the capture / replay of a
// step (native/runtime/decode_executor.cpp:163-209).  Attention, RoPE/KV and sampling
// beyond greedy are not part of it: the attention block is stood in for by taking the
// first `hidden` features of the fused qkv output.
#include <cstring>
#include <new>

#include "common.cuh"
#include "decode_chain.cuh"
#include "gemv_rows.cuh"
#include "skinny_gemm.cuh"

#include <atomic>
#include <vector>

namespace mcl {

enum : uint32_t {
    SEC_QKV = 0, SEC_O = 1, SEC_GATE_UP = 2, SEC_DOWN = 3, SEC_NORM1 = 4, SEC_NORM2 = 5,
    SEC_QKV_SCALE = 6, SEC_O_SCALE = 7, SEC_GATE_UP_SCALE = 8, SEC_DOWN_SCALE = 9,
    SEC_LM_HEAD = 10, SEC_FINAL_NORM = 11, SEC_LM_HEAD_SCALE = 12, SEC_COUNT = 13
};

static inline size_t align256(size_t v) { return (v + 255u) & ~(size_t)255u; }

struct Layout {
    size_t per_layer[10];      // byte size of SEC_QKV .. SEC_DOWN_SCALE (0 when absent)
    size_t layer_off[10];      // offset inside one layer block
    size_t layer_bytes;        // pitch of a layer block
    size_t top_off[3], top_bytes[3];   // lm_head, final_norm, lm_head_scale
    size_t total;
};

// Rows [lo, lo + rows) of an n-row tensor owned by `rank`; pitch = ceil(n / world) rounded up to 8.
struct Span { uint32_t lo, rows, pitch; };
static Span shard_span(uint32_t n, uint32_t world, uint32_t rank) {
    if (world <= 1u) return {0u, n, n};
    const uint32_t pitch = ((n + world - 1u) / world + 7u) & ~7u;
    const uint32_t lo = rank * pitch < n ? rank * pitch : n;
    return {lo, (n - lo < pitch ? n - lo : pitch), pitch};
}
static uint32_t world_of(const mc_sm100_stack_desc_t* d) { return d->world <= 1u ? 1u : d->world; }

static bool valid_desc(const mc_sm100_stack_desc_t* d) {
    if (d == nullptr || d->struct_size != sizeof(mc_sm100_stack_desc_t)) return false;
    if (d->layers == 0 || d->layers > 4096u || d->hidden == 0 || d->qkv_rows < d->hidden || d->inter == 0 || d->vocab == 0) return false;
    if (d->precision != 0u && d->precision != 2u) return false;
    if (d->max_batch == 0 || d->max_batch > 64u) return false;
    const uint32_t mult = d->precision == 2u ? 16u : 8u;
    if (d->hidden % mult != 0 || d->inter % mult != 0) return false;
    if (d->reserved[0] != 0 || d->reserved[1] != 0) return false;
    if (d->world > 8u || (d->world > 1u && d->rank >= d->world) || (d->world <= 1u && d->rank != 0)) return false;
    if (d->world > 1u) {
        // every rank owns at least one row of every layer linear
        const uint32_t w = d->world;
        if (shard_span(d->qkv_rows, w, w - 1u).rows == 0 || shard_span(d->hidden, w, w - 1u).rows == 0 ||
            shard_span(d->inter, w, w - 1u).rows == 0 || shard_span(d->vocab, w, w - 1u).rows == 0)
            return false;
    }
    return true;
}

static Layout make_layout(const mc_sm100_stack_desc_t* d) {
    Layout L{};
    const size_t wb = d->precision == 2u ? 1u : 2u;
    const uint32_t W = world_of(d), R = d->rank;
    const size_t H = d->hidden, I = d->inter;
    // rows of this rank's shard (the whole tensor on one GPU)
    const size_t Q = shard_span(d->qkv_rows, W, R).rows, Ho = shard_span(d->hidden, W, R).rows,
                 Ip = shard_span(d->inter, W, R).rows, V = shard_span(d->vocab, W, R).rows;
    const bool fp8 = d->precision == 2u;
    const size_t sizes[10] = {Q * H * wb, Ho * H * wb, 2 * Ip * H * wb, Ho * I * wb, H * 2, H * 2,
                              fp8 ? Q * 4 : 0, fp8 ? Ho * 4 : 0, fp8 ? 2 * Ip * 4 : 0, fp8 ? Ho * 4 : 0};
    size_t off = 0;
    for (int i = 0; i < 10; ++i) {
        L.per_layer[i] = sizes[i];
        L.layer_off[i] = off;
        off += align256(sizes[i]);
    }
    L.layer_bytes = off;
    size_t top = L.layer_bytes * d->layers;
    const size_t tops[3] = {V * H * wb, H * 2, fp8 ? V * 4 : 0};
    for (int i = 0; i < 3; ++i) {
        L.top_off[i] = top;
        L.top_bytes[i] = tops[i];
        top += align256(tops[i]);
    }
    L.total = top;
    return L;
}

// activation scratch (bf16 unless noted), all 256-byte aligned
struct Scratch {
    size_t x, res_a, res_b, h, qkv, ctx, o, mid, down, logits, stage, tokens, vals, sync, total;
    // one-launch M = 1 chain (one GPU): its table of linears (64 bytes each), their arrival counters and the
    // four tagged vectors (qkv, o, mid, down: one 32-bit word per element) the linears hand to one another
    size_t chain_table, chain_arrivals, chain_buf[4];
};

static Scratch make_scratch(const mc_sm100_stack_desc_t* d) {
    Scratch s{};
    const size_t M = d->max_batch, H = d->hidden;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t at = off; off += align256(bytes); return at; };
    s.x = take(M * H * 2); s.res_a = take(M * H * 2); s.res_b = take(M * H * 2); s.h = take(M * H * 2);
    s.qkv = take(M * d->qkv_rows * 2); s.ctx = take(M * H * 2); s.o = take(M * H * 2);
    s.mid = take(M * (size_t)d->inter * 2); s.down = take(M * H * 2); s.logits = take(M * (size_t)d->vocab * 2);
    s.stage = take(mc_sm100_argmax_stage_bytes(d->max_batch)); s.tokens = take(M * 4); s.vals = take(M * 4);
    s.sync = take(1024);  // words [0] count of M = 1 sharded steps + 1 (the exchange tags derive from it), [1] failure word
                          // (bounded waits of any kernel of a step), [2] shard token, [3] shard value, [5] gather epoch,
                          // [6] count of batched sharded steps + 1; peer address tables (8 x u64 each) at bytes 64 pairs,
                          // 128 pair counters of M = 1 steps, 192 pair counters of batched steps, 256.. batched buffers
                          // [7] count of batched sharded steps whose GEMMs do the exchange themselves + 1,
                          // [8] count of one-launch M = 1 steps + 1, [9] arrival ticket of that kernel's token reduction
    s.chain_table = take(((size_t)d->layers * 4 + 1) * 64);
    s.chain_arrivals = take(((size_t)d->layers * 4 + 1) * 4);
    const size_t cdims[4] = {d->qkv_rows, H, d->inter, H};
    for (int k = 0; k < 4; ++k) s.chain_buf[k] = take(cdims[k] * 4);
    s.total = off;
    return s;
}

// Exchange region of a sharded stack, identical on every rank: the four gathered vectors of
// a layer (tagged 32-bit words), then the (value, index) pairs of the greedy reduction and
// their arrival counters.
enum : uint32_t { XK_QKV = 0, XK_O = 1, XK_MID = 2, XK_DOWN = 3, XK_VECS = 4 };
struct Exchange {
    size_t buf[XK_VECS];     // gathered qkv, o, mid, down (tagged words, M = 1)
    uint32_t pitch[XK_VECS]; // slot pitch in elements (the same for the batched buffers)
    size_t pairs, pair_flags;   // [8][max_batch] x 8 bytes; 8 x uint32 for M = 1 steps, then 8 x uint32 for batched steps
    // batched steps (M > 1): plain bf16 [max_batch, full width] activations + the gather's arrival flags
    size_t bbuf[XK_VECS], bflags;
    size_t tbuf[XK_VECS];    // the same four activations as tagged 64-bit words (two bf16 + a 32-bit sequence number), written by the GEMMs themselves
    uint32_t width[XK_VECS];
    size_t bytes;
};
static Exchange make_exchange(const mc_sm100_stack_desc_t* d) {
    Exchange x{};
    const uint32_t W = world_of(d);
    const uint32_t dims[XK_VECS] = {d->qkv_rows, d->hidden, d->inter, d->hidden};
    size_t off = 0;
    for (uint32_t k = 0; k < XK_VECS; ++k) {
        x.pitch[k] = shard_span(dims[k], W, 0).pitch;
        x.width[k] = dims[k];
        x.buf[k] = off;
        off += align256((size_t)x.pitch[k] * W * 4u);
    }
    x.pairs = off; off += align256(8u * 8u * (size_t)d->max_batch);
    x.pair_flags = off; off += align256(16u * 4u);
    if (d->max_batch > 1u) {
        for (uint32_t k = 0; k < XK_VECS; ++k) { x.bbuf[k] = off; off += align256((size_t)d->max_batch * dims[k] * 2u); }
        x.bflags = off; off += align256(8u * 4u);
        for (uint32_t k = 0; k < XK_VECS; ++k) { x.tbuf[k] = off; off += align256((size_t)d->max_batch * dims[k] * 4u); }
    }
    x.bytes = off;
    return x;
}

}  // namespace mcl

using namespace mcl;

struct mc_sm100_stack {
    Exchange xch;
    uint64_t peer[8];              // exchange regions of all ranks as mapped here (0 = not bound)
    uint64_t timeout_ns;
    mc_sm100_stack_desc_t desc;
    Layout lay;
    Scratch scr;
    uint8_t* w;
    uint8_t* s;
    cudaGraphExec_t graph[65];     // per batch size, captured lazily
    cudaStream_t graph_stream[65];
    int32_t* h_status;             // pinned host word the failure word is read into after a host step
    uint32_t chain_slot;           // ring slot size of the one-launch M = 1 chain; 0 = shapes do not fit, per-linear kernels
    uint32_t chain_kmax;
    uint32_t chain_nshapes, chain_shape_rows[CHAIN_SHAPES], chain_shape_gran[CHAIN_SHAPES], chain_shape_rpu[CHAIN_SHAPES];
};

// 1: an M = 1 step of a one-GPU stack is one persistent kernel; 0 (default): one kernel per linear.  Measured on
// the benchmark's 40-layer stream: 1.245 ms against 1.097 ms (bf16), 1.219 against 0.892 ms (e4m3): the
// hand-over of a vector between the CTAs costs ~2 us per linear and the ring then refills in bursts.
static std::atomic<int> g_chain_mode{0};

// Weights of section `which` of layer `layer` as a prefetch hint for the launch that follows.
static void hint(const mc_sm100_stack* st, uint32_t layer, uint32_t which);

static const void* sec(const mc_sm100_stack* st, uint32_t layer, uint32_t which) {
    if (which < 10) return st->lay.per_layer[which] ? st->w + st->lay.layer_bytes * layer + st->lay.layer_off[which] : nullptr;
    return st->lay.top_bytes[which - 10] ? st->w + st->lay.top_off[which - 10] : nullptr;
}

static void hint(const mc_sm100_stack* st, uint32_t layer, uint32_t which) {
    const size_t bytes = which < 10 ? st->lay.per_layer[which] : st->lay.top_bytes[which - 10];
    mc_sm100_hint_next_weights(sec(st, layer, which), bytes);
}

// Sharded M = 1 step: the fused chain with every output exchanged inside the GEMV kernels.
// Exchange kind k happens once per layer; its sequence number in step s (from 1), layer l is
// (s - 1) * layers + l + 1.  Every rank carries the whole residual stream redundantly.
static mc_status_t run_step_sharded(mc_sm100_stack* st, const uint16_t* d_x, int32_t* d_tokens, cudaStream_t stream) {
    const mc_sm100_stack_desc_t& d = st->desc;
    const uint32_t W = d.world, R = d.rank, H = d.hidden, I = d.inter, L = d.layers;
    if (st->peer[R] == 0) { set_error("stack step: sharded stack without a bound exchange region"); return MC_E_INVALID_ARGUMENT; }
    const bool fp8 = d.precision == 2u;
    const Exchange& x = st->xch;
    const uint64_t own = st->peer[R];
    const uint32_t rows_q = shard_span(d.qkv_rows, W, R).rows, rows_h = shard_span(H, W, R).rows,
                   rows_i = shard_span(I, W, R).rows;
    const Span sv = shard_span(d.vocab, W, R);
    uint32_t* sync = reinterpret_cast<uint32_t*>(st->s + st->scr.sync);
    auto buf = [&](size_t off) { return reinterpret_cast<uint16_t*>(st->s + off); };
    uint16_t *ra = buf(st->scr.res_a), *rb = buf(st->scr.res_b), *logits = buf(st->scr.logits);
    // gathered vectors are uint32 words; the sharded entry points take them through their bf16 pointer arguments
    auto gathered = [&](uint32_t k) { return reinterpret_cast<const uint16_t*>(own + x.buf[k]); };
    // consume: exchange kind read by this linear (-1: local input) and its number within the step;
    // produce: kind written (-1: output stays local) and its number
    auto io = [&](int consume, uint32_t in_add, int produce, uint32_t out_add) {
        mc_sm100_shard_io_t o{};
        o.struct_size = sizeof(o); o.world = W; o.rank = R;
        o.d_step = sync; o.d_status = reinterpret_cast<int32_t*>(sync + 1); o.timeout_ns = st->timeout_ns;
        if (consume >= 0) { o.in_tagged = 1; o.in_seq_mul = L; o.in_seq_add = in_add; }
        if (produce >= 0) {
            o.out_slot = x.pitch[produce]; o.out_seq_mul = L; o.out_seq_add = out_add;
            for (uint32_t p = 0; p < W; ++p) o.out_peer[p] = st->peer[p] + x.buf[produce];
        }
        return o;
    };
    void* sp = (void*)stream;
    mc_status_t rc = MC_OK;
#define STEP(call) do { rc = (call); if (rc != MC_OK) return rc; } while (0)
    const uint16_t* res_in = d_x;
    for (uint32_t l = 0; l < L; ++l) {
        const uint16_t *n1 = (const uint16_t*)sec(st, l, SEC_NORM1), *n2 = (const uint16_t*)sec(st, l, SEC_NORM2);
        const float* no_scale = nullptr;
        auto scale = [&](uint32_t which) { return fp8 ? (const float*)sec(st, l, which) : no_scale; };
        mc_sm100_shard_io_t q = io(l == 0 ? -1 : (int)XK_DOWN, l, XK_QKV, l + 1);
        hint(st, l, SEC_O);
        STEP(mc_sm100_gemv_sharded(1, 0, sec(st, l, SEC_QKV), scale(SEC_QKV_SCALE), res_in, l == 0 ? nullptr : gathered(XK_DOWN),
                                   n1, rb, nullptr, rows_q, H, d.eps, &q, sp, 1));
        q = io(XK_QKV, l + 1, XK_O, l + 1);
        hint(st, l, SEC_GATE_UP);
        STEP(mc_sm100_gemv_sharded(0, 0, sec(st, l, SEC_O), scale(SEC_O_SCALE), gathered(XK_QKV), nullptr, nullptr, nullptr,
                                   nullptr, rows_h, H, d.eps, &q, sp, 1));
        q = io(XK_O, l + 1, XK_MID, l + 1);
        hint(st, l, SEC_DOWN);
        STEP(mc_sm100_gemv_sharded(1, 1, sec(st, l, SEC_GATE_UP), scale(SEC_GATE_UP_SCALE), rb, gathered(XK_O), n2, ra, nullptr,
                                   2u * rows_i, H, d.eps, &q, sp, 1));
        q = io(XK_MID, l + 1, XK_DOWN, l + 1);
        if (l + 1 < L) hint(st, l + 1, SEC_QKV); else hint(st, 0, SEC_LM_HEAD);
        STEP(mc_sm100_gemv_sharded(0, 0, sec(st, l, SEC_DOWN), scale(SEC_DOWN_SCALE), gathered(XK_MID), nullptr, nullptr, nullptr,
                                   nullptr, rows_h, I, d.eps, &q, sp, 1));
        res_in = ra;
    }
    const mc_sm100_shard_io_t q = io(XK_DOWN, L, -1, 0);
    float* shard_val = reinterpret_cast<float*>(sync + 3);
    int32_t* shard_tok = reinterpret_cast<int32_t*>(sync + 2);
    hint(st, 0, SEC_QKV);      // the next step starts with layer 0 again
    STEP(mc_sm100_lm_head_argmax_sharded(sec(st, 0, SEC_LM_HEAD), (const float*)sec(st, 0, SEC_LM_HEAD_SCALE), res_in,
                                         gathered(XK_DOWN), (const uint16_t*)sec(st, 0, SEC_FINAL_NORM), rb, logits, sv.rows, H,
                                         d.eps, (int32_t)sv.lo, st->s + st->scr.stage, shard_tok, shard_val, &q, sp, 1));
    STEP(mc_sm100_peer_argmax(shard_val, shard_tok, 1u, reinterpret_cast<const uint64_t*>(sync + 16),
                              reinterpret_cast<const uint64_t*>(sync + 32), reinterpret_cast<const uint64_t*>(own + x.pairs),
                              reinterpret_cast<const uint32_t*>(own + x.pair_flags), sync, R, W, st->timeout_ns,
                              reinterpret_cast<int32_t*>(sync + 1), d_tokens, reinterpret_cast<float*>(st->s + st->scr.vals), sp, 1));
#undef STEP
    return MC_OK;
}

// A bf16 batched linear inside a step: the tcgen05 kernel wherever it takes the shape -- also at the row counts where
// the public entry point would pick the register-streaming mma.sync kernel (see linear_cols) -- else the public entry
// point's CUDA-core fallback.
static mc_status_t stack_gemm_bf16(const void* w, const uint16_t* x, uint16_t* y, uint32_t M, uint32_t N, uint32_t K, cudaStream_t stream) {
    if (M >= 2u && mcl::skinny_shape_ok(N, K, 2))
        return mcl::skinny_gemm(mcl::SKINNY_W_BF16, w, nullptr, x, nullptr, y, M, N, K, false, stream, true);
    return mc_sm100_gemm_bf16((void*)stream, nullptr, 0, M, N, K, w, x, y);
}

// o_proj of a batched step: its activation is the first `hidden` columns of the [M, pitch] qkv
// result (the stand-in for attention).  The tensor-core GEMM reads that column block in place
// through its tensor map; the CUDA-core forms (fewest rows, shapes TMA cannot take) get a packed copy.
static mc_status_t linear_cols(mc_sm100_stack* st, uint32_t M, uint32_t l, const uint16_t* src, uint32_t pitch, uint16_t* ctx,
                               uint16_t* y, uint32_t rows, cudaStream_t stream) {
    const mc_sm100_stack_desc_t& d = st->desc;
    const bool fp8 = d.precision == 2u;
    const uint32_t H = d.hidden;
    const void* w = sec(st, l, SEC_O);
    const float* sc = fp8 ? (const float*)sec(st, l, SEC_O_SCALE) : nullptr;
    const bool tensor = (fp8 ? M >= 4u : M >= 2u) && mcl::skinny_shape_ok(rows, H, fp8 ? 1 : 2) && (pitch & 7u) == 0u;
    // (the tcgen05 kernel also at the row counts where the register-streaming mma.sync kernel wins a chain of identical
    // calls: between tensor-core kernels of two CTAs per SM that one-CTA-per-SM kernel cannot become resident early, and
    // the M = 8 step was measured at 2.11 ms with it against 1.91 ms)
    if (tensor)
        return mcl::skinny_gemm(fp8 ? mcl::SKINNY_W_E4M3 : mcl::SKINNY_W_BF16, w, sc, src, nullptr, y, M, rows, H, false, stream, true, pitch);
    const cudaError_t e = cudaMemcpy2DAsync(ctx, (size_t)H * 2, src, (size_t)pitch * 2, (size_t)H * 2, M, cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) { mcl::set_error("stack step: copy failed: %s", cudaGetErrorString(e)); return MC_E_CUDA; }
    return fp8 ? mc_sm100_gemv_fp8_rows_m((const uint8_t*)w, sc, ctx, y, M, rows, H, (void*)stream, 1)
               : mc_sm100_gemm_bf16((void*)stream, nullptr, 0, M, rows, H, w, ctx, y);
}

// Sharded batched step (M > 1): every rank runs the batched chain on its rows of each matrix; the
// [M, rows] result of a linear is scattered into column slot `rank` of every rank's [M, width]
// buffer by one small kernel per linear (mc_sm100_peer_allgather_rows), which is then the activation
// of the next GEMM.  The residual stream and the norms are computed redundantly on every rank.
static mc_status_t run_step_sharded_batched(mc_sm100_stack* st, const uint16_t* d_x, uint32_t M, int32_t* d_tokens, cudaStream_t stream) {
    const mc_sm100_stack_desc_t& d = st->desc;
    const uint32_t W = d.world, R = d.rank, H = d.hidden, I = d.inter, L = d.layers;
    if (st->peer[R] == 0) { set_error("stack step: sharded stack without a bound exchange region"); return MC_E_INVALID_ARGUMENT; }
    if ((d.qkv_rows | H | I) & 7u) { set_error("stack step: sharded batched steps need widths that are multiples of 8"); return MC_E_UNSUPPORTED; }
    const bool fp8 = d.precision == 2u;
    const Exchange& x = st->xch;
    const uint64_t own = st->peer[R];
    const Span sq = shard_span(d.qkv_rows, W, R), sh = shard_span(H, W, R), si = shard_span(I, W, R), sv = shard_span(d.vocab, W, R);
    uint32_t* sync = reinterpret_cast<uint32_t*>(st->s + st->scr.sync);
    uint8_t* sync_b = reinterpret_cast<uint8_t*>(sync);
    int32_t* status = reinterpret_cast<int32_t*>(sync + 1);
    auto buf = [&](size_t off) { return reinterpret_cast<uint16_t*>(st->s + off); };
    uint16_t *ra = buf(st->scr.res_a), *h = buf(st->scr.h), *ctx = buf(st->scr.ctx), *logits = buf(st->scr.logits);
    uint16_t* part = buf(I >= d.qkv_rows ? st->scr.mid : st->scr.qkv);      // this rank's [M, rows] result of the current linear
    auto full = [&](uint32_t k) { return reinterpret_cast<uint16_t*>(own + x.bbuf[k]); };
    void* sp = (void*)stream;
    mc_status_t rc = MC_OK;
#define STEP(call) do { rc = (call); if (rc != MC_OK) return rc; } while (0)
    // this rank's [M, rows] result (contiguous in `part`) -> column slot of every rank's buffer k
    auto gather = [&](uint32_t k, uint32_t rows) {
        return mc_sm100_peer_allgather_rows(part, M, rows * 2u, x.width[k] * 2u, x.pitch[k] * 2u,
                                            reinterpret_cast<const uint64_t*>(sync_b + 256u + 64u * k),
                                            reinterpret_cast<const uint64_t*>(sync_b + 512u),
                                            reinterpret_cast<uint32_t*>(own + x.bflags), sync + 5, R, W, st->timeout_ns, status, sp, 1);
    };
    auto linear = [&](uint32_t l, uint32_t wsec, uint32_t ssec, const uint16_t* in, uint32_t rows, uint32_t K) {
        return fp8 ? mc_sm100_gemv_fp8_rows_m((const uint8_t*)sec(st, l, wsec), (const float*)sec(st, l, ssec), in, part, M, rows, K, sp, 1)
                   : stack_gemm_bf16(sec(st, l, wsec), in, part, M, rows, K, stream);
    };
    // When every linear of the layer runs on the tensor cores, the GEMM itself stores its result into every rank's
    // buffer, as tagged words (two bf16 + the exchange's 32-bit sequence number; no fence, no flag).  The norms read
    // their addend from those words; the two GEMMs whose activation is such a buffer (o_proj, down_proj) get it
    // through a small kernel that polls the tags and writes plain bf16 for the TMA loads.  No gather kernels.
    const int mode = fp8 ? SKINNY_W_E4M3 : SKINNY_W_BF16;
    const int wbytes = fp8 ? 1 : 2;
    const bool fused = (fp8 ? M >= 4u : M >= 2u) && skinny_shape_ok(sq.rows, H, wbytes) && skinny_shape_ok(sh.rows, H, wbytes) &&
                       skinny_shape_ok(2u * si.rows, H, wbytes) && skinny_shape_ok(sh.rows, I, wbytes);
    if (fused) {
        uint16_t* mid_plain = buf(st->scr.mid);
        auto out_of = [&](uint32_t k, uint32_t lsel) {
            PeerOut o{};
            for (uint32_t p = 0; p < W; ++p) o.base[p] = st->peer[p] + x.tbuf[k];
            o.step = sync + 7; o.world = W; o.pitch = x.width[k] / 2u; o.col0 = R * x.pitch[k] / 2u; o.layers = L; o.lsel = lsel;
            return o;
        };
        auto in_of = [&](uint32_t k, uint32_t lsel) {
            TaggedIn t{};
            t.words = reinterpret_cast<const uint64_t*>(own + x.tbuf[k]);
            t.step = sync + 7; t.pitch = x.width[k] / 2u; t.layers = L; t.lsel = lsel;
            t.timeout_ns = st->timeout_ns ? st->timeout_ns : kShardWaitDefaultNs; t.status = status;
            return t;
        };
        auto gemm = [&](uint32_t l, uint32_t wsec, uint32_t ssec, const uint16_t* in, uint32_t rows, uint32_t K, bool swiglu, uint32_t out_kind) {
            const PeerOut o = out_of(out_kind, l + 1u);
            return skinny_gemm(mode, sec(st, l, wsec), fp8 ? (const float*)sec(st, l, ssec) : nullptr, in, nullptr, part, M, rows, K, swiglu,
                               stream, true, 0, &o);
        };
        cudaError_t ce = cudaMemcpyAsync(ra, d_x, (size_t)M * H * 2, cudaMemcpyDeviceToDevice, stream);
        if (ce != cudaSuccess) { set_error("stack step: copy failed: %s", cudaGetErrorString(ce)); return MC_E_CUDA; }
        for (uint32_t l = 0; l < L; ++l) {
            // exchange numbers within the step: kind k of layer l is number l + 1 of its kind
            STEP(residual_rmsnorm_rows_tagged(ra, nullptr, (const uint16_t*)sec(st, l, SEC_NORM1), h, M, H, d.eps,
                                              l == 0 ? TaggedIn{} : in_of(XK_DOWN, l), nullptr, stream, true));
            hint(st, l, SEC_O);
            STEP(gemm(l, SEC_QKV, SEC_QKV_SCALE, h, sq.rows, H, false, XK_QKV));
            STEP(detag_rows(in_of(XK_QKV, l + 1u), ctx, M, H, stream, true));        // attention stand-in: the first H columns of qkv
            hint(st, l, SEC_GATE_UP);
            STEP(gemm(l, SEC_O, SEC_O_SCALE, ctx, sh.rows, H, false, XK_O));
            STEP(residual_rmsnorm_rows_tagged(ra, nullptr, (const uint16_t*)sec(st, l, SEC_NORM2), h, M, H, d.eps, in_of(XK_O, l + 1u), nullptr, stream, true));
            hint(st, l, SEC_DOWN);
            STEP(gemm(l, SEC_GATE_UP, SEC_GATE_UP_SCALE, h, 2u * si.rows, H, true, XK_MID));
            STEP(detag_rows(in_of(XK_MID, l + 1u), mid_plain, M, I, stream, true));
            if (l + 1 < L) hint(st, l + 1, SEC_QKV); else hint(st, 0, SEC_LM_HEAD);
            STEP(gemm(l, SEC_DOWN, SEC_DOWN_SCALE, mid_plain, sh.rows, I, false, XK_DOWN));
        }
        // the last norm also moves the step word on: every kernel of this step has read it by then
        STEP(residual_rmsnorm_rows_tagged(ra, nullptr, (const uint16_t*)sec(st, 0, SEC_FINAL_NORM), h, M, H, d.eps, in_of(XK_DOWN, L), sync + 7, stream, true));
    } else {
    cudaError_t e = cudaMemcpyAsync(ra, d_x, (size_t)M * H * 2, cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) { set_error("stack step: copy failed: %s", cudaGetErrorString(e)); return MC_E_CUDA; }
    const uint16_t* addend = nullptr;
    for (uint32_t l = 0; l < L; ++l) {
        STEP(mc_sm100_residual_rmsnorm_rows(ra, addend, (const uint16_t*)sec(st, l, SEC_NORM1), h, M, H, d.eps, sp, 1));
        hint(st, l, SEC_O);
        STEP(linear(l, SEC_QKV, SEC_QKV_SCALE, h, sq.rows, H));
        STEP(gather(XK_QKV, sq.rows));
        hint(st, l, SEC_GATE_UP);
        STEP(linear_cols(st, M, l, full(XK_QKV), x.width[XK_QKV], ctx, part, sh.rows, stream));
        STEP(gather(XK_O, sh.rows));
        STEP(mc_sm100_residual_rmsnorm_rows(ra, full(XK_O), (const uint16_t*)sec(st, l, SEC_NORM2), h, M, H, d.eps, sp, 1));
        hint(st, l, SEC_DOWN);
        STEP(mc_sm100_gate_up_swiglu(sec(st, l, SEC_GATE_UP), (const float*)sec(st, l, SEC_GATE_UP_SCALE), h, part, M, 2u * si.rows, H, sp, 1));
        STEP(gather(XK_MID, si.rows));
        if (l + 1 < L) hint(st, l + 1, SEC_QKV); else hint(st, 0, SEC_LM_HEAD);
        STEP(linear(l, SEC_DOWN, SEC_DOWN_SCALE, full(XK_MID), sh.rows, I));
        STEP(gather(XK_DOWN, sh.rows));
        addend = full(XK_DOWN);
    }
    STEP(mc_sm100_residual_rmsnorm_rows(ra, addend, (const uint16_t*)sec(st, 0, SEC_FINAL_NORM), h, M, H, d.eps, sp, 1));
    }
    void* stage = st->s + st->scr.stage;
    int32_t* shard_tok = reinterpret_cast<int32_t*>(st->s + st->scr.tokens);
    float* shard_val = reinterpret_cast<float*>(st->s + st->scr.vals);
    hint(st, 0, SEC_QKV);      // the next step starts with layer 0 again
    if (M <= 8u) {
        STEP(mc_sm100_lm_head_argmax(sec(st, 0, SEC_LM_HEAD), (const float*)sec(st, 0, SEC_LM_HEAD_SCALE), h, logits, sv.rows, M, sv.rows, H,
                                     (int32_t)sv.lo, stage, shard_tok, shard_val, sp, 1));
    } else {
        rc = fp8 ? mc_sm100_gemv_fp8_rows_m((const uint8_t*)sec(st, 0, SEC_LM_HEAD), (const float*)sec(st, 0, SEC_LM_HEAD_SCALE), h, logits, M, sv.rows, H, sp, 1)
                 : stack_gemm_bf16(sec(st, 0, SEC_LM_HEAD), h, logits, M, sv.rows, H, stream);
        if (rc != MC_OK) return rc;
        STEP(mc_sm100_argmax_bf16(logits, M, sv.rows, sv.rows, (int32_t)sv.lo, stage, shard_tok, shard_val, sp, 1));
    }
    // per-row (value, index) of every rank -> tokens; the winning values land in the (otherwise unused) o scratch
    // its own step word and arrival counters: the M = 1 exchange tags count M = 1 steps only, so a
    // run of batched steps can never bring a stale tag back into range
    STEP(mc_sm100_peer_argmax(shard_val, shard_tok, M, reinterpret_cast<const uint64_t*>(sync + 16), reinterpret_cast<const uint64_t*>(sync + 48),
                              reinterpret_cast<const uint64_t*>(own + x.pairs), reinterpret_cast<const uint32_t*>(own + x.pair_flags + 32u), sync + 6, R, W,
                              st->timeout_ns, status, d_tokens, reinterpret_cast<float*>(st->s + st->scr.o), sp, 1));
#undef STEP
    return MC_OK;
}

static mc_status_t run_step_inner(mc_sm100_stack* st, const uint16_t* d_x, uint32_t M, int32_t* d_tokens, cudaStream_t stream);

// One step for M rows; every launch goes to `stream`, nothing synchronises.  For its duration the
// bounded waits of every kernel launched from this thread report into the stack's failure word.
static mc_status_t run_step(mc_sm100_stack* st, const uint16_t* d_x, uint32_t M, int32_t* d_tokens, cudaStream_t stream) {
    set_wait_status_sink(reinterpret_cast<int32_t*>(st->s + st->scr.sync) + 1);
    const mc_status_t rc = run_step_inner(st, d_x, M, d_tokens, stream);
    set_wait_status_sink(nullptr);
    mc_sm100_hint_next_weights(nullptr, 0);     // a step that failed half way must not leave a hint behind
    return rc;
}

static mc_status_t run_step_inner(mc_sm100_stack* st, const uint16_t* d_x, uint32_t M, int32_t* d_tokens, cudaStream_t stream) {
    const mc_sm100_stack_desc_t& d = st->desc;
    const uint32_t H = d.hidden, Q = d.qkv_rows, I = d.inter, V = d.vocab;
    const bool fp8 = d.precision == 2u;
    auto buf = [&](size_t off) { return reinterpret_cast<uint16_t*>(st->s + off); };
    uint16_t *ra = buf(st->scr.res_a), *rb = buf(st->scr.res_b), *h = buf(st->scr.h), *qkv = buf(st->scr.qkv),
             *ctx = buf(st->scr.ctx), *o = buf(st->scr.o), *mid = buf(st->scr.mid), *dn = buf(st->scr.down),
             *logits = buf(st->scr.logits);
    void* stage = st->s + st->scr.stage;
    float* vals = reinterpret_cast<float*>(st->s + st->scr.vals);
    void* sp = (void*)stream;
    mc_status_t rc = MC_OK;
    if (d.world > 1u) return M == 1 ? run_step_sharded(st, d_x, d_tokens, stream) : run_step_sharded_batched(st, d_x, M, d_tokens, stream);
#define STEP(call) do { rc = (call); if (rc != MC_OK) return rc; } while (0)
    if (M == 1 && st->chain_slot != 0u && g_chain_mode.load(std::memory_order_relaxed) != 0) {
        uint32_t* sync = reinterpret_cast<uint32_t*>(st->s + st->scr.sync);
        ChainArgs a{};
        a.table = reinterpret_cast<const ChainLinear*>(st->s + st->scr.chain_table);
        a.count = 4u * d.layers + 1u;
        a.H = H; a.kmax = st->chain_kmax; a.slot_bytes = st->chain_slot;
        a.nshapes = st->chain_nshapes;
        for (uint32_t i = 0; i < CHAIN_SHAPES; ++i) {
            a.shape_rows[i] = st->chain_shape_rows[i]; a.shape_gran[i] = st->chain_shape_gran[i]; a.shape_rpu[i] = st->chain_shape_rpu[i];
        }
        for (int k = 0; k < 4; ++k) a.bufs[k] = reinterpret_cast<uint32_t*>(st->s + st->scr.chain_buf[k]);
        a.arrivals = reinterpret_cast<uint32_t*>(st->s + st->scr.chain_arrivals);
        a.x_in = d_x; a.logits = logits;
        a.stage_val = reinterpret_cast<float*>(stage);
        a.stage_idx = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(stage) + 4096);
        a.token = d_tokens; a.token_val = vals;
        a.step = sync + 8; a.ticket = sync + 9; a.status = reinterpret_cast<int32_t*>(sync + 1);
        a.timeout_ns = st->timeout_ns ? st->timeout_ns : kShardWaitDefaultNs;
        a.eps = d.eps;
        return decode_chain_launch(fp8 ? 1 : 2, a, stream);
    }
    if (M == 1) {
        // fused chain: residual add + RMSNorm live in the GEMV prologues, SwiGLU in the gate_up epilogue
        const uint16_t* res_in = d_x;
        const uint16_t* addend = nullptr;
        for (uint32_t l = 0; l < d.layers; ++l) {
            const uint16_t *n1 = (const uint16_t*)sec(st, l, SEC_NORM1), *n2 = (const uint16_t*)sec(st, l, SEC_NORM2);
            // every launch is told which weights the launch after it will stream (L2 prefetch)
            hint(st, l, SEC_O);
            if (fp8) STEP(mc_sm100_gemv_fp8_prologue((const uint8_t*)sec(st, l, SEC_QKV), (const float*)sec(st, l, SEC_QKV_SCALE), res_in, addend, n1, rb, qkv, Q, H, d.eps, sp, 1));
            else STEP(mc_sm100_gemv_rows_prologue((const uint16_t*)sec(st, l, SEC_QKV), res_in, addend, n1, rb, qkv, Q, H, d.eps, sp, 1));
            hint(st, l, SEC_GATE_UP);
            if (fp8) STEP(mc_sm100_gemv_fp8((const uint8_t*)sec(st, l, SEC_O), (const float*)sec(st, l, SEC_O_SCALE), qkv, o, H, H, sp, 1));
            else STEP(mc_sm100_decode_gemv((const uint16_t*)sec(st, l, SEC_O), qkv, o, H, H, MC_GEMV_TACTIC_ROWS, 0, nullptr, sp, 1));
            hint(st, l, SEC_DOWN);
            STEP(mc_sm100_gate_up_swiglu_prologue(sec(st, l, SEC_GATE_UP), (const float*)sec(st, l, SEC_GATE_UP_SCALE), rb, o, n2, ra, mid, 2 * I, H, d.eps, sp, 1));
            if (l + 1 < d.layers) hint(st, l + 1, SEC_QKV); else hint(st, 0, SEC_LM_HEAD);
            if (fp8) STEP(mc_sm100_gemv_fp8((const uint8_t*)sec(st, l, SEC_DOWN), (const float*)sec(st, l, SEC_DOWN_SCALE), mid, dn, H, I, sp, 1));
            else STEP(mc_sm100_decode_gemv((const uint16_t*)sec(st, l, SEC_DOWN), mid, dn, H, I, MC_GEMV_TACTIC_ROWS, 0, nullptr, sp, 1));
            res_in = ra;
            addend = dn;
        }
        hint(st, 0, SEC_QKV);      // the next step starts with layer 0 again
        STEP(mc_sm100_lm_head_argmax_prologue(sec(st, 0, SEC_LM_HEAD), (const float*)sec(st, 0, SEC_LM_HEAD_SCALE), res_in, addend,
                                              (const uint16_t*)sec(st, 0, SEC_FINAL_NORM), rb, logits, V, H, d.eps, 0, stage,
                                              d_tokens, vals, sp, 1));
        return MC_OK;
    }
    // batched chain: separate residual+RMSNorm kernels between the tensor-core GEMMs
    cudaError_t e = cudaMemcpyAsync(ra, d_x, (size_t)M * H * 2, cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) { set_error("stack step: copy failed: %s", cudaGetErrorString(e)); return MC_E_CUDA; }
    auto linear = [&](uint32_t l, uint32_t wsec, uint32_t ssec, const uint16_t* x, uint16_t* y, uint32_t N, uint32_t K) {
        return fp8 ? mc_sm100_gemv_fp8_rows_m((const uint8_t*)sec(st, l, wsec), (const float*)sec(st, l, ssec), x, y, M, N, K, sp, 1)
                   : stack_gemm_bf16(sec(st, l, wsec), x, y, M, N, K, stream);
    };
    const uint16_t* addend = nullptr;
    for (uint32_t l = 0; l < d.layers; ++l) {
        STEP(mc_sm100_residual_rmsnorm_rows(ra, addend, (const uint16_t*)sec(st, l, SEC_NORM1), h, M, H, d.eps, sp, 1));
        hint(st, l, SEC_O);
        STEP(linear(l, SEC_QKV, SEC_QKV_SCALE, h, qkv, Q, H));
        hint(st, l, SEC_GATE_UP);
        STEP(linear_cols(st, M, l, qkv, Q, ctx, o, H, stream));
        STEP(mc_sm100_residual_rmsnorm_rows(ra, o, (const uint16_t*)sec(st, l, SEC_NORM2), h, M, H, d.eps, sp, 1));
        hint(st, l, SEC_DOWN);
        STEP(mc_sm100_gate_up_swiglu(sec(st, l, SEC_GATE_UP), (const float*)sec(st, l, SEC_GATE_UP_SCALE), h, mid, M, 2 * I, H, sp, 1));
        if (l + 1 < d.layers) hint(st, l + 1, SEC_QKV); else hint(st, 0, SEC_LM_HEAD);
        STEP(linear(l, SEC_DOWN, SEC_DOWN_SCALE, mid, dn, H, I));
        addend = dn;
    }
    STEP(mc_sm100_residual_rmsnorm_rows(ra, addend, (const uint16_t*)sec(st, 0, SEC_FINAL_NORM), h, M, H, d.eps, sp, 1));
    hint(st, 0, SEC_QKV);      // the next step starts with layer 0 again
    if (M <= 8) {
        STEP(mc_sm100_lm_head_argmax(sec(st, 0, SEC_LM_HEAD), (const float*)sec(st, 0, SEC_LM_HEAD_SCALE), h, logits, V, M, V, H, 0, stage, d_tokens, vals, sp, 1));
    } else {
        STEP(linear(0, SEC_LM_HEAD, SEC_LM_HEAD_SCALE, h, logits, V, H));
        STEP(mc_sm100_argmax_bf16(logits, M, V, V, 0, stage, d_tokens, vals, sp, 1));
    }
#undef STEP
    return MC_OK;
}

// The table of the one-launch M = 1 chain: per layer qkv (residual + norm prologue), o, gate_up (residual + norm
// prologue, SwiGLU epilogue), down, then the lm_head (final norm, greedy token).  Leaves chain_slot 0 when the
// shapes do not fit the kernel's shared memory or its argmax staging.
static cudaError_t chain_setup(mc_sm100_stack* st) {
    const mc_sm100_stack_desc_t& d = st->desc;
    const bool fp8 = d.precision == 2u;
    const int wb = fp8 ? 1 : 2;
    const uint32_t H = d.hidden, I = d.inter;
    const uint32_t kmax = H > I ? H : I;
    const uint32_t unit_max = (2u * H > I ? 2u * H : I) * (uint32_t)wb;      // a gate/up pair, or one down row
    if ((uint32_t)sm_count() * 8u > 4096u || mc_sm100_argmax_stage_bytes(1) < 8192u) return cudaSuccess;
    const uint32_t slot = chain_slot_bytes(wb, H, kmax, unit_max);
    if (slot == 0u) return cudaSuccess;
    std::vector<ChainLinear> t;
    bool too_many = false;
    uint32_t nshapes = 0, srows[CHAIN_SHAPES] = {0}, sgran[CHAIN_SHAPES] = {1, 1, 1, 1, 1, 1, 1, 1}, srpu[CHAIN_SHAPES] = {1, 1, 1, 1, 1, 1, 1, 1};
    auto add = [&](uint32_t l, uint32_t wsec, uint32_t ssec, uint32_t nsec, uint32_t N, uint32_t K, uint32_t pro, uint32_t epi,
                   uint32_t in_buf, uint32_t out_buf) {
        ChainLinear c{};
        c.w = reinterpret_cast<const uint8_t*>(sec(st, l, wsec));
        c.scale = fp8 ? reinterpret_cast<const float*>(sec(st, l, ssec)) : nullptr;
        c.norm_w = pro == PRO_RESNORM ? reinterpret_cast<const uint16_t*>(sec(st, l, nsec)) : nullptr;
        c.N = N; c.K = K; c.pro = pro; c.epi = epi; c.in_buf = in_buf; c.out_buf = out_buf;
        c.rows_per_unit = chain_rows_per_unit(wb, K, epi, slot);
        const uint32_t gran = epi == EPI_SWIGLU ? 2u : 1u;
        uint32_t sid = 0;
        while (sid < nshapes && !(srows[sid] == N && sgran[sid] == gran && srpu[sid] == c.rows_per_unit)) ++sid;
        if (sid == nshapes && nshapes < CHAIN_SHAPES) { srows[sid] = N; sgran[sid] = gran; srpu[sid] = c.rows_per_unit; ++nshapes; }
        c.shape = sid;
        too_many = too_many || sid >= CHAIN_SHAPES;
        t.push_back(c);
    };
    for (uint32_t l = 0; l < d.layers; ++l) {
        add(l, SEC_QKV, SEC_QKV_SCALE, SEC_NORM1, d.qkv_rows, H, PRO_RESNORM, EPI_STORE, l == 0 ? CHAIN_IN_X : 3u, 0u);
        add(l, SEC_O, SEC_O_SCALE, 0, H, H, PRO_NONE, EPI_STORE, 0u, 1u);       // activation: the first H words of qkv
        add(l, SEC_GATE_UP, SEC_GATE_UP_SCALE, SEC_NORM2, 2u * I, H, PRO_RESNORM, EPI_SWIGLU, 1u, 2u);
        add(l, SEC_DOWN, SEC_DOWN_SCALE, 0, H, I, PRO_NONE, EPI_STORE, 2u, 3u);
    }
    add(0, SEC_LM_HEAD, SEC_LM_HEAD_SCALE, SEC_FINAL_NORM, d.vocab, H, PRO_RESNORM, EPI_ARGMAX, 3u, CHAIN_IN_NONE);
    if (too_many) return cudaSuccess;
    cudaError_t e = cudaMemcpy(st->s + st->scr.chain_table, t.data(), t.size() * sizeof(ChainLinear), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(st->s + st->scr.chain_arrivals, 0, t.size() * 4);
    for (int k = 0; k < 4 && e == cudaSuccess; ++k) {
        const size_t dims[4] = {d.qkv_rows, H, I, H};
        e = cudaMemset(st->s + st->scr.chain_buf[k], 0, dims[k] * 4);       // tag 0: not what the first steps wait for
    }
    if (e == cudaSuccess) {
        st->chain_slot = slot; st->chain_kmax = kmax; st->chain_nshapes = nshapes;
        for (uint32_t i = 0; i < CHAIN_SHAPES; ++i) { st->chain_shape_rows[i] = srows[i]; st->chain_shape_gran[i] = sgran[i]; st->chain_shape_rpu[i] = srpu[i]; }
    }
    return e;
}

extern "C" {

void mc_sm100_debug_set_chain(int32_t on) { g_chain_mode.store(on != 0 ? 1 : 0, std::memory_order_relaxed); }

mc_status_t mc_sm100_stack_sizes(const mc_sm100_stack_desc_t* desc, uint64_t* weight_bytes, uint64_t* scratch_bytes) {
    clear_error();
    if (!valid_desc(desc)) { set_error("mc_sm100_stack_sizes: invalid descriptor"); return MC_E_INVALID_ARGUMENT; }
    if (weight_bytes) *weight_bytes = make_layout(desc).total;
    if (scratch_bytes) *scratch_bytes = make_scratch(desc).total;
    return MC_OK;
}

mc_status_t mc_sm100_stack_section(const mc_sm100_stack_desc_t* desc, uint32_t layer, uint32_t which, uint64_t* offset,
                                   uint64_t* bytes) {
    clear_error();
    if (!valid_desc(desc) || which >= SEC_COUNT || (which < 10 && layer >= desc->layers) || offset == nullptr || bytes == nullptr) {
        set_error("mc_sm100_stack_section: invalid args (layer=%u which=%u)", layer, which);
        return MC_E_INVALID_ARGUMENT;
    }
    const Layout L = make_layout(desc);
    if (which < 10) { *offset = L.layer_bytes * layer + L.layer_off[which]; *bytes = L.per_layer[which]; }
    else { *offset = L.top_off[which - 10]; *bytes = L.top_bytes[which - 10]; }
    return MC_OK;
}

mc_status_t mc_sm100_stack_create(const mc_sm100_stack_desc_t* desc, void* d_weights, void* d_scratch,
                                  mc_sm100_stack_t* out) {
    clear_error();
    if (out != nullptr) *out = nullptr;
    if (!valid_desc(desc) || d_weights == nullptr || d_scratch == nullptr || out == nullptr ||
        ((uintptr_t)d_weights & 255u) != 0 || ((uintptr_t)d_scratch & 255u) != 0) {
        set_error("mc_sm100_stack_create: invalid args (descriptor, or arenas not 256-byte aligned)");
        return MC_E_INVALID_ARGUMENT;
    }
    const mc_status_t dc = mc_sm100_device_check(nullptr, nullptr, nullptr, nullptr);
    if (dc != MC_OK) return dc;
    mc_sm100_stack* st = new (std::nothrow) mc_sm100_stack();
    if (st == nullptr) { set_error("mc_sm100_stack_create: out of host memory"); return MC_E_OUT_OF_MEMORY; }
    st->desc = *desc;
    st->lay = make_layout(desc);
    st->scr = make_scratch(desc);
    st->w = (uint8_t*)d_weights;
    st->s = (uint8_t*)d_scratch;
    st->xch = make_exchange(desc);
    std::memset(st->peer, 0, sizeof(st->peer));
    st->timeout_ns = 0;
    std::memset(st->graph, 0, sizeof(st->graph));
    std::memset(st->graph_stream, 0, sizeof(st->graph_stream));
    st->h_status = nullptr;
    // control words of the scratch arena: step counters 1, failure word 0 (a sharded stack sets
    // them again, with its peer tables, when the exchange region is bound)
    uint32_t words[256] = {0};
    words[0] = 1u; words[6] = 1u; words[7] = 1u; words[8] = 1u;
    cudaError_t e = cudaMemcpy(st->s + st->scr.sync, words, sizeof(words), cudaMemcpyHostToDevice);
    st->chain_slot = 0;
    st->chain_kmax = 0;
    if (e == cudaSuccess && world_of(desc) == 1u) e = chain_setup(st);
    if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&st->h_status), 64, cudaHostAllocDefault);
    if (e != cudaSuccess) {
        set_error("mc_sm100_stack_create: %s", cudaGetErrorString(e));
        if (st->h_status != nullptr) cudaFreeHost(st->h_status);
        delete st;
        return MC_E_CUDA;
    }
    *st->h_status = 0;
    *out = st;
    return MC_OK;
}

mc_status_t mc_sm100_stack_exchange_bytes(const mc_sm100_stack_desc_t* desc, uint64_t* bytes) {
    clear_error();
    if (!valid_desc(desc) || bytes == nullptr) { set_error("mc_sm100_stack_exchange_bytes: invalid descriptor"); return MC_E_INVALID_ARGUMENT; }
    *bytes = desc->world > 1u ? make_exchange(desc).bytes : 0u;
    return MC_OK;
}

mc_status_t mc_sm100_stack_bind_exchange(mc_sm100_stack_t st, const uint64_t* h_peer_addrs, uint64_t timeout_ns, void* stream) {
    clear_error();
    if (st == nullptr || h_peer_addrs == nullptr || st->desc.world <= 1u) {
        set_error("mc_sm100_stack_bind_exchange: invalid args (not a sharded stack?)");
        return MC_E_INVALID_ARGUMENT;
    }
    const uint32_t W = st->desc.world, R = st->desc.rank;
    for (uint32_t p = 0; p < W; ++p)
        if (h_peer_addrs[p] == 0 || (h_peer_addrs[p] & 255u) != 0) {
            set_error("mc_sm100_stack_bind_exchange: address of rank %u missing or not 256-byte aligned", p);
            return MC_E_INVALID_ARGUMENT;
        }
    // graphs captured against an earlier binding hold its addresses
    for (auto& g : st->graph)
        if (g != nullptr) { cudaGraphExecDestroy(g); g = nullptr; }
    const cudaStream_t s = (cudaStream_t)stream;
    uint32_t words[256] = {0};
    words[0] = 1u;   // step counters start at 1; [1] failure word = 0; [5] gather epoch = 0
    words[6] = 1u; words[7] = 1u; words[8] = 1u;
    uint64_t* tables = reinterpret_cast<uint64_t*>(words + 16);          // byte 64: pairs, byte 128 / 192: pair counters (M = 1 / batched)
    uint64_t* btables = reinterpret_cast<uint64_t*>(words + 64);         // byte 256 + 64 k: batched buffer k; byte 512: gather flags
    for (uint32_t p = 0; p < W; ++p) {
        st->peer[p] = h_peer_addrs[p];
        tables[p] = h_peer_addrs[p] + st->xch.pairs;
        tables[8 + p] = h_peer_addrs[p] + st->xch.pair_flags;
        tables[16 + p] = h_peer_addrs[p] + st->xch.pair_flags + 32u;
        if (st->desc.max_batch > 1u) {
            for (uint32_t k = 0; k < XK_VECS; ++k) btables[8u * k + p] = h_peer_addrs[p] + st->xch.bbuf[k];
            btables[8u * XK_VECS + p] = h_peer_addrs[p] + st->xch.bflags;
        }
    }
    st->timeout_ns = timeout_ns;
    cudaError_t e = cudaMemsetAsync(reinterpret_cast<void*>(st->peer[R]), 0, st->xch.bytes, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(st->s + st->scr.sync, words, sizeof(words), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { set_error("mc_sm100_stack_bind_exchange: %s", cudaGetErrorString(e)); return MC_E_CUDA; }
    return MC_OK;
}

mc_status_t mc_sm100_stack_exchange_status(mc_sm100_stack_t st, int32_t* h_status, void* stream) {
    clear_error();
    if (st == nullptr || h_status == nullptr) { set_error("mc_sm100_stack_exchange_status: invalid args"); return MC_E_INVALID_ARGUMENT; }
    const cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(h_status, st->s + st->scr.sync + 4, 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { set_error("mc_sm100_stack_exchange_status: %s", cudaGetErrorString(e)); return MC_E_CUDA; }
    return MC_OK;
}

void mc_sm100_stack_destroy(mc_sm100_stack_t st) {
    if (st == nullptr) return;
    for (auto& g : st->graph)
        if (g != nullptr) cudaGraphExecDestroy(g);
    if (st->h_status != nullptr) cudaFreeHost(st->h_status);
    delete st;
}

const int32_t* mc_sm100_stack_status_word(mc_sm100_stack_t st) {
    return st == nullptr ? nullptr : reinterpret_cast<const int32_t*>(st->s + st->scr.sync) + 1;
}

const uint16_t* mc_sm100_stack_logits(mc_sm100_stack_t st) {
    return st == nullptr ? nullptr : reinterpret_cast<const uint16_t*>(st->s + st->scr.logits);
}

mc_status_t mc_sm100_stack_step(mc_sm100_stack_t st, const uint16_t* d_x, uint32_t M, int32_t* d_tokens, void* stream) {
    clear_error();
    if (st == nullptr || d_x == nullptr || d_tokens == nullptr || M == 0 || M > st->desc.max_batch) {
        set_error("mc_sm100_stack_step: invalid args (M=%u)", M);
        return MC_E_INVALID_ARGUMENT;
    }
    return run_step(st, d_x, M, d_tokens, (cudaStream_t)stream);
}

mc_status_t mc_sm100_stack_step_host(mc_sm100_stack_t st, const uint16_t* h_x, uint32_t M, int32_t* h_tokens, void* stream) {
    clear_error();
    if (st == nullptr || h_x == nullptr || h_tokens == nullptr || M == 0 || M > st->desc.max_batch) {
        set_error("mc_sm100_stack_step_host: invalid args (M=%u)", M);
        return MC_E_INVALID_ARGUMENT;
    }
    const cudaStream_t s = (cudaStream_t)stream;
    uint16_t* d_x = reinterpret_cast<uint16_t*>(st->s + st->scr.x);
    int32_t* d_tok = reinterpret_cast<int32_t*>(st->s + st->scr.tokens);
    cudaError_t e = cudaMemcpyAsync(d_x, h_x, (size_t)M * st->desc.hidden * 2, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) { set_error("stack step: H2D failed: %s", cudaGetErrorString(e)); return MC_E_CUDA; }
    mc_status_t rc = MC_OK;
    bool done = false;
    if (st->desc.enable_cuda_graph && s != nullptr) {
        if (st->graph[M] == nullptr || st->graph_stream[M] != s) {
            // first use of this batch size on this stream: THIS call's step runs eagerly (it also sets
            // the kernel attributes), then the same sequence is captured -- a capture launches nothing --
            // for the calls that follow.  A failed capture leaves eager launches of the same kernels
            // (the reference does the same, native/runtime/session.cpp:489-499).
            rc = run_step(st, d_x, M, d_tok, s);
            if (rc != MC_OK) return rc;
            done = true;
            cudaGraph_t g = nullptr;
            if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
                const mc_status_t cap = run_step(st, d_x, M, d_tok, s);
                const cudaError_t ce = cudaStreamEndCapture(s, &g);
                if (cap == MC_OK && ce == cudaSuccess && g != nullptr) {
                    if (st->graph[M] != nullptr) cudaGraphExecDestroy(st->graph[M]);
                    st->graph[M] = nullptr;
                    if (cudaGraphInstantiate(&st->graph[M], g, 0) == cudaSuccess) st->graph_stream[M] = s;
                    else st->graph[M] = nullptr;
                }
                if (g != nullptr) cudaGraphDestroy(g);
                (void)cudaGetLastError();
            }
        }
        if (!done && st->graph[M] != nullptr) {
            e = cudaGraphLaunch(st->graph[M], s);
            if (e != cudaSuccess) { set_error("stack step: graph launch failed: %s", cudaGetErrorString(e)); return MC_E_GRAPH; }
            done = true;
        }
    }
    if (!done) rc = run_step(st, d_x, M, d_tok, s);
    if (rc != MC_OK) return rc;
    e = cudaMemcpyAsync(h_tokens, d_tok, (size_t)M * 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(st->h_status, st->s + st->scr.sync + 4, 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { set_error("stack step: D2H/sync failed: %s", cudaGetErrorString(e)); return MC_E_CUDA; }
    if (*st->h_status != 0) {
        set_error("stack step: a bounded wait ran out inside a kernel (a peer rank is gone or out of step, or a tensor-core "
                  "pipeline stalled); the tokens of this step are undefined");
        return MC_E_INTERNAL;
    }
    return MC_OK;
}

}  // extern "C"
