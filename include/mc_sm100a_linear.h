/* mc_sm100a_linear.h -- C ABI of the B200 (sm_100a) decode linear-layer library.
 *
 * This is the drop-in boundary for ONE path of the reference runtime: the
 * decode-time linear layers (M=1 GEMV in bf16 and in e4m3 weight-only with a
 * per-output-row fp32 scale, the fused variants around them, and the M<=64
 * batched-decode skinny GEMM).  Every entry point below replaces one internal
 * launcher / engine method of the reference; the citation beside each one is
 * the reference interface it stands in for (path relative to the reference
 * project root).  Argument order, meaning and error behaviour follow the
 * reference; shape restrictions of the reference (hidden size fixed at 2048,
 * M capped at 8, ...) are lifted.
 *
 * Conventions (same as native/include/minicpm_runtime.h:1-12 and
 * native/kernels/sm120/kernels.h:3-11):
 *   - extern "C", fixed-width integers, plain pointers; no CUDA or C++ types
 *     in signatures.  `stream` is a cudaStream_t passed as void* (NULL = the
 *     legacy default stream).  bf16 travels as raw uint16_t bit patterns,
 *     e4m3 as uint8_t codes.
 *   - every pointer named d_* is DEVICE memory; h_* is HOST memory.
 *   - every call returns mc_status_t; on failure an English message is left
 *     in a thread-local buffer readable through mc_last_error().
 *   - no call allocates device memory, synchronises, or takes a host-side
 *     decision that depends on device data unless its comment says so: the
 *     launch shapes depend only on the arguments, so a sequence of calls can
 *     be captured into a CUDA graph and replayed.
 *   - `pdl` != 0 launches with programmatic stream serialisation; the kernels
 *     then issue their weight loads before griddepcontrol.wait and release
 *     their dependents at entry, like the reference kernels do
 *     (native/kernels/sm120/kernels.h:25-57).
 *   - there is no CPU and no library-GEMM fallback behind any of these.
 */
#ifndef MC_SM100A_LINEAR_H
#define MC_SM100A_LINEAR_H

#include <stddef.h>
#include <stdint.h>

/* Only the entry points below are exported from the shared library (hidden
 * visibility otherwise, as native/runtime/export.h does for MC_API). */
#if defined(__GNUC__)
#define MC_SM100_API __attribute__((visibility("default")))
#else
#define MC_SM100_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: numerically identical to native/include/minicpm_runtime.h:34-44. */
#ifndef MC_STATUS_T_DEFINED
#define MC_STATUS_T_DEFINED
typedef enum mc_status_t {
    MC_OK = 0,
    MC_E_INVALID_ARGUMENT = 1,
    MC_E_IO = 2,
    MC_E_CUDA = 3,
    MC_E_MODEL_MISMATCH = 4,
    MC_E_OUT_OF_MEMORY = 5,
    MC_E_GRAPH = 6,
    MC_E_UNSUPPORTED = 7,
    MC_E_INTERNAL = 100
} mc_status_t;
#endif

/* GEMV tactics: values of native/kernels/sm120/kernels.h:109-117.  Tactic 0
 * (library GEMM) does not exist here and is rejected. */
#define MC_GEMV_TACTIC_ROWS   1
#define MC_GEMV_TACTIC_SPLITK 2
#define MC_GEMV_TACTIC_FP8    3

/* Thread-local diagnostic of the last failing call on this thread
 * (native/include/minicpm_runtime.h:131; native/runtime/error.cpp:14-41). */
MC_SM100_API const char* mc_sm100_last_error(void);

/* Library / device probe.  Fills sm_count, L2 bytes and compute capability of
 * the CURRENT device; MC_E_UNSUPPORTED unless it is compute capability 10.x
 * (stands where the reference checks for 12.0, native/runtime/model.cpp:133-139). */
MC_SM100_API mc_status_t mc_sm100_device_check(int32_t* out_sm_count, uint64_t* out_l2_bytes,
                                  int32_t* out_cc_major, int32_t* out_cc_minor);

/* Names the weights that the linear AFTER the next one will stream (any device range,
 * 16-byte aligned).  When the L2 prefetch is switched on (mc_sm100_debug_set_prefetch; it is
 * OFF by default) the next streaming launch made by the calling thread (GEMV, batched GEMM)
 * asks the memory system, while it runs, to bring that range from HBM into L2
 * (cp.async.bulk.prefetch.L2 or prefetch.global.L2).  The hint is consumed by that one launch;
 * ranges beyond 64 MB are cut.  No counterpart in the reference; the caller that knows the
 * chain is the executor (native/runtime/forward.cpp:206-462), and mc_sm100_stack_step names
 * the next weights for every linear of its chain.  Measured on B200 the prefetch does not
 * pay (the prefetched lines are mostly evicted before the next kernel reads them, and an L2
 * hit streams only ~1.5 x faster than HBM), which is why it is off; the plumbing stays for
 * parts where it does.  A call with NULL clears a pending hint.  Results never depend on it. */
MC_SM100_API void mc_sm100_hint_next_weights(const void* d_next_w, uint64_t bytes);

/* ---------------------------------------------------------------- M = 1 ---- */

/* y[N] = bf16( W[N,K] . x[K] ), fp32 accumulate, one rounding.
 * Replaces launch_decode_gemv (native/kernels/sm120/kernels.h:666-672,
 * native/kernels/sm120/gemv.cu:382-431).  W row-major, 16-byte aligned,
 * K % 8 == 0.  tactic ROWS: one pass.  tactic SPLITK: K is cut into split_s
 * equal segments ((K/split_s) % 8 == 0), fp32 partials [split_s, N] go to
 * d_split_partial and are merged in fixed order (no atomics: bit-reproducible). */
MC_SM100_API mc_status_t mc_sm100_decode_gemv(const uint16_t* d_w, const uint16_t* d_x, uint16_t* d_y,
                                 uint32_t N, uint32_t K, int32_t tactic, uint32_t split_s,
                                 float* d_split_partial, void* stream, int32_t pdl);

/* Tactic of one shape, fixed once and used for every later call (select_decode_gemv_tactics /
 * run_decode_gemv, native/runtime/gemv_tactic.cpp:91-258; gemv_tactic.h:42-90): the row kernel
 * is timed against split-K with S = 8, 4, 2 on the current device, on the caller's weights, and
 * the winner is returned (a split has to be 3 % faster: its sums run in another order).  The
 * library-GEMM candidate of the reference does not exist here.  With d_flush (>= twice the L2)
 * the weights come from HBM in every timed call; without it they stay L2-resident as in the
 * reference's timing loop.  Synchronises the stream; a load-time call.  d_partial needs
 * mc_sm100_gemv_partial_floats(max N) floats (NULL: only the row kernel is timed). */
typedef struct mc_sm100_gemv_tactic_t {
    uint32_t struct_size;
    int32_t  tactic;            /* MC_GEMV_TACTIC_ROWS or MC_GEMV_TACTIC_SPLITK */
    uint32_t split_s;           /* 1 for ROWS */
    uint32_t best_split_s;      /* fastest split tried (0: none applied) */
    float    us_rows, us_splitk;/* median microseconds of the row kernel and of the fastest split */
    uint32_t reserved[2];
} mc_sm100_gemv_tactic_t;
MC_SM100_API uint32_t mc_sm100_gemv_pick_split_s(uint32_t N, uint32_t K);   /* the reference's static rule, target = 2 CTAs per SM of this device */
MC_SM100_API size_t mc_sm100_gemv_partial_floats(uint32_t max_n);
MC_SM100_API mc_status_t mc_sm100_select_decode_gemv_tactic(const uint16_t* d_w, uint32_t N, uint32_t K, const uint16_t* d_x,
                                                            uint16_t* d_y, float* d_partial, size_t partial_floats,
                                                            void* d_flush, size_t flush_bytes, void* stream,
                                                            mc_sm100_gemv_tactic_t* out);
MC_SM100_API mc_status_t mc_sm100_run_decode_gemv(const mc_sm100_gemv_tactic_t* tactic, const uint16_t* d_w,
                                                  const uint16_t* d_x, uint16_t* d_y, uint32_t N, uint32_t K,
                                                  float* d_partial, void* stream, int32_t pdl);

/* Split-K bf16 GEMV for callers that cannot allocate device memory (a frozen
 * arena, a step replayed from a graph, a plugin host without an allocator).
 * This entry point has no counterpart in the reference.  Same arithmetic and
 * result as mc_sm100_decode_gemv with tactic SPLITK, but the fp32 partials live
 * in a 512 KiB array that is part of the library image, so split_s * N must
 * not exceed 131072 (MC_E_UNSUPPORTED otherwise).  It calls no allocator of
 * any kind.  The first call on each device looks the array's address up
 * (cudaGetSymbolAddress, that device current); make that call before any stream
 * capture.  All calls share the one array: two calls that overlap on the GPU
 * (different streams, or the same graph replayed concurrently) race; calls
 * ordered on one stream are safe, and no call depends on what an earlier call
 * left in the array. */
MC_SM100_API mc_status_t mc_sm100_decode_gemv_splitk_static(const uint16_t* d_w, const uint16_t* d_x,
                                                            uint16_t* d_y, uint32_t N, uint32_t K,
                                                            uint32_t split_s, void* stream, int32_t pdl);

/* y[N] = bf16( scale[n] * sum_k e4m3(W[n,k]) * x[k] ); the row scale multiplies
 * the finished fp32 sum once.  Replaces launch_gemv_fp8
 * (native/kernels/sm120/kernels.h:721-726, gemv_fp8.cu:694-721).  Any K; the
 * vector path needs K % 16 == 0 and 16-byte aligned W and x, everything else
 * takes a byte-wise path with the same arithmetic.  Codes 0x7F/0xFF decode to
 * +/-480 like the reference's bit decoder (kernels.h:120-125). */
MC_SM100_API mc_status_t mc_sm100_gemv_fp8(const uint8_t* d_w, const float* d_scale, const uint16_t* d_x,
                              uint16_t* d_y, uint32_t N, uint32_t K, void* stream, int32_t pdl);

/* Fused prologue: res_out = bf16(res_in + addend) (addend may be NULL: plain
 * copy), h = rmsnorm(res_out) * norm_w, y = W . h.  The normalised vector
 * stays on chip.  Replace launch_gemv_rows_prologue / launch_gemv_fp8_prologue
 * (native/kernels/sm120/kernels.h:735-748, gemv.cu:148-246, gemv_fp8.cu:213-315);
 * `n` (= K of the GEMV) is no longer fixed at 2048.  res_in/res_out must be
 * different buffers (the reference ping-pongs them, forward.cpp:206-237). */
MC_SM100_API mc_status_t mc_sm100_gemv_rows_prologue(const uint16_t* d_w, const uint16_t* d_res_in,
                                        const uint16_t* d_addend, const uint16_t* d_norm_w,
                                        uint16_t* d_res_out, uint16_t* d_y, uint32_t N,
                                        uint32_t n, float eps, void* stream, int32_t pdl);
MC_SM100_API mc_status_t mc_sm100_gemv_fp8_prologue(const uint8_t* d_w, const float* d_scale,
                                       const uint16_t* d_res_in, const uint16_t* d_addend,
                                       const uint16_t* d_norm_w, uint16_t* d_res_out,
                                       uint16_t* d_y, uint32_t N, uint32_t n, float eps,
                                       void* stream, int32_t pdl);

/* Down projection with the SwiGLU computed on the way in:
 * h[k] = bf16( silu(gate_up[k]) * gate_up[K+k] ), y = W[N,K] . h.
 * Replace launch_gemv_rows_swiglu / launch_gemv_fp8_swiglu
 * (native/kernels/sm120/kernels.h:753-764); K is no longer fixed at 6144. */
MC_SM100_API mc_status_t mc_sm100_gemv_rows_swiglu(const uint16_t* d_w, const uint16_t* d_gate_up,
                                      uint16_t* d_y, uint32_t N, uint32_t K, void* stream,
                                      int32_t pdl);
MC_SM100_API mc_status_t mc_sm100_gemv_fp8_swiglu(const uint8_t* d_w, const float* d_scale,
                                     const uint16_t* d_gate_up, uint16_t* d_y, uint32_t N,
                                     uint32_t K, void* stream, int32_t pdl);

/* Fused gate_up projection with a SwiGLU EPILOGUE (the B200 arena layout):
 * the weight holds gate and up rows interleaved (row 2j = gate_j, row 2j+1 =
 * up_j; see mc_sm100_interleave_rows), N = 2*I rows in total, and
 * y[m, j] = bf16( silu(bf16 g) * bf16 u ) with g/u the bf16-ROUNDED dot
 * products -- bit-compatible with running the plain GEMV and then
 * swiglu_gated_kernel (native/kernels/sm120/swiglu.cu:57-70;
 * tools/reference_forward.py:293-294).  d_scale == NULL selects bf16 weights
 * (d_w read as uint16_t), otherwise e4m3 weights with interleaved row scales.
 * M in [1,64] (CUDA cores up to 4 rows, tcgen05 above); x [M,K], y [M, N/2]. */
MC_SM100_API mc_status_t mc_sm100_gate_up_swiglu(const void* d_w_interleaved, const float* d_scale_interleaved,
                                    const uint16_t* d_x, uint16_t* d_y, uint32_t M, uint32_t N,
                                    uint32_t K, void* stream, int32_t pdl);

/* The same with the residual-add + RMSNorm prologue in front (M = 1): what the
 * reference does for gate_up with launch_gemv_*_prologue followed by the
 * SwiGLU of the down projection (native/runtime/forward.cpp:306-373), in one
 * kernel on the interleaved layout.  y [N/2]. */
MC_SM100_API mc_status_t mc_sm100_gate_up_swiglu_prologue(
    const void* d_w_interleaved, const float* d_scale_interleaved, const uint16_t* d_res_in,
    const uint16_t* d_addend, const uint16_t* d_norm_w, uint16_t* d_res_out, uint16_t* d_y,
    uint32_t N, uint32_t n, float eps, void* stream, int32_t pdl);

/* Arena re-layout helper for the call above: dst row 2j = src row j, dst row
 * 2j+1 = src row I+j, for rows of row_bytes bytes (weights) -- call it again
 * with row_bytes = 4 for the fp32 scales.  Runs on the device, src != dst. */
MC_SM100_API mc_status_t mc_sm100_interleave_rows(const void* d_src, void* d_dst, uint32_t I,
                                     uint32_t row_bytes, void* stream);

/* ------------------------------------------------------------ 2 <= M <= 64 -- */

/* y[M,N] = bf16( scale[n] * sum_k e4m3(W[n,k]) * x[m,k] ), weight-only fp8.
 * Replaces launch_gemv_fp8_rows_m (native/kernels/sm120/kernels.h:774-779),
 * whose cap of M <= 8 becomes M <= 64.  M <= 3 runs on CUDA cores and every
 * output row is bit-equal to the M=1 call on that row; larger M dequantises
 * e4m3 -> bf16 (exact) on the way into shared memory and uses tcgen05 MMA. */
MC_SM100_API mc_status_t mc_sm100_gemv_fp8_rows_m(const uint8_t* d_w, const float* d_scale,
                                     const uint16_t* d_x, uint16_t* d_y, uint32_t M,
                                     uint32_t N, uint32_t K, void* stream, int32_t pdl);

/* C[M,N] = bf16( B[M,K] . A[N,K]^T ): d_a is the WEIGHT [N,K], d_b the
 * activation [M,K], both row-major (operand order of GemmEngine::gemm_bf16,
 * native/runtime/gemm.h:3-11, 61-63; native/runtime/gemm.cpp:316-380).
 * M in [1,64].  workspace: kept for signature compatibility (the reference
 * passes its 16 MB per-session workspace here); split-K partials are reduced
 * through distributed shared memory inside a thread-block cluster, so
 * mc_sm100_gemm_workspace_bytes returns 0 and NULL is accepted. */
MC_SM100_API mc_status_t mc_sm100_gemm_bf16(void* stream, void* d_workspace, size_t ws_size, uint32_t M,
                               uint32_t N, uint32_t K, const void* d_a, const void* d_b,
                               void* d_c);
MC_SM100_API size_t mc_sm100_gemm_workspace_bytes(uint32_t M, uint32_t N, uint32_t K);

/* W8A8 form of the batched GEMM (GemmEngine::gemm_fp8_q / gemm_fp8,
 * native/runtime/gemm.h:64-90): Y = (Wq*w_scale[n]) . (Xq*x_scale[m])^T with
 * tcgen05 kind::f8f6f4.  gemm_fp8 quantises the bf16 activation per row first
 * (launch_quant_rows, native/kernels/sm120/quant.cu:98-136) into the caller's
 * scratch.  This is NOT the weight-only arithmetic: it is judged against the
 * quantisation-aware CPU statement. */
MC_SM100_API mc_status_t mc_sm100_gemm_fp8_q(void* stream, void* d_workspace, size_t ws_size, uint32_t M,
                                uint32_t N, uint32_t K, const void* d_w_fp8,
                                const float* d_w_scale, const void* d_x_fp8,
                                const float* d_x_scale, uint16_t* d_y_bf16);
MC_SM100_API mc_status_t mc_sm100_gemm_fp8(void* stream, void* d_workspace, size_t ws_size, uint32_t M,
                              uint32_t N, uint32_t K, const void* d_w_fp8, const float* d_w_scale,
                              const uint16_t* d_x_bf16, uint16_t* d_y_bf16,
                              void* d_x_fp8_scratch, float* d_x_scale_scratch);

/* bf16 [M,K] -> e4m3 [M,K] + scale[M] (amax/448; all-zero row -> scale 1), and
 * y[m,n] *= w_scale[n]*x_scale[m] (x_scale may be NULL).  Replace
 * launch_quant_rows / launch_post_scale_rows (kernels.h:785-798). */
MC_SM100_API mc_status_t mc_sm100_quant_rows(const uint16_t* d_x, uint8_t* d_xq, float* d_scale, uint32_t M,
                                uint32_t K, void* stream);
MC_SM100_API mc_status_t mc_sm100_post_scale_rows(uint16_t* d_y, const float* d_w_scale,
                                     const float* d_x_scale, uint32_t M, uint32_t N,
                                     void* stream);

/* Batched residual add + RMSNorm between the batched GEMMs: res[r,:] =
 * bf16(res + add) in place (add may be NULL), out[r,:] = bf16(res * rsqrt(mean
 * (res^2) + eps) * w) on the rounded residual.  The M = 1 chain has this fused
 * into the GEMV prologue; the batched chain calls it like the reference's
 * BatchGroup does (launch_residual_add_rmsnorm, native/kernels/sm120/rmsnorm.cu:130-166;
 * native/runtime/batch_group.cpp:770, 794). */
MC_SM100_API mc_status_t mc_sm100_residual_rmsnorm_rows(uint16_t* d_res, const uint16_t* d_add,
                                                        const uint16_t* d_norm_w, uint16_t* d_out,
                                                        uint32_t rows, uint32_t n, float eps,
                                                        void* stream, int32_t pdl);

/* ------------------------------------------------------- lm_head / greedy --- */

/* Greedy argmax over bf16 logits compared as fp32, ties to the lowest index,
 * rows [n_rows, vocab]; writes one int32 per row.  Two-stage; d_stage needs
 * mc_sm100_argmax_stage_bytes(n_rows) bytes.  Replaces
 * launch_sampling_greedy_bf16 / launch_batch_argmax_bf16
 * (native/kernels/sm120/sampling.cu:637-685, 186-234).  index_base is added
 * to the indices (vocab shards); d_out_val (optional) receives the winning
 * value as fp32 so that shards can be compared across ranks. */
MC_SM100_API mc_status_t mc_sm100_argmax_bf16(const uint16_t* d_logits, uint32_t n_rows, uint32_t vocab,
                                 uint32_t row_stride, int32_t index_base, void* d_stage,
                                 int32_t* d_out_idx, float* d_out_val, void* stream,
                                 int32_t pdl);
MC_SM100_API size_t mc_sm100_argmax_stage_bytes(uint32_t n_rows);

/* lm_head GEMV (bf16 weights when d_scale == NULL, else e4m3 + row scales) for
 * M in [1,8] rows with the per-shard argmax fused behind it: logits [M,N] are
 * written (row stride y_stride elements) and (value, index_base + index) of
 * each row's maximum go to d_out_val / d_out_idx.  N need not be a multiple
 * of anything (vocab 122753).  Stands for the reference's lm_head GEMV +
 * two-stage argmax pair (native/runtime/forward.cpp:443-489). */
MC_SM100_API mc_status_t mc_sm100_lm_head_argmax(const void* d_w, const float* d_scale, const uint16_t* d_x,
                                    uint16_t* d_logits, uint32_t y_stride, uint32_t M,
                                    uint32_t N, uint32_t K, int32_t index_base, void* d_stage,
                                    int32_t* d_out_idx, float* d_out_val, void* stream,
                                    int32_t pdl);

/* The same for M = 1 with the final residual-add + RMSNorm in front (the
 * reference runs lm_head through launch_gemv_fp8_prologue,
 * native/runtime/forward.cpp:443-462). */
MC_SM100_API mc_status_t mc_sm100_lm_head_argmax_prologue(
    const void* d_w, const float* d_scale, const uint16_t* d_res_in, const uint16_t* d_addend,
    const uint16_t* d_norm_w, uint16_t* d_res_out, uint16_t* d_logits, uint32_t N, uint32_t n,
    float eps, int32_t index_base, void* d_stage, int32_t* d_out_idx, float* d_out_val,
    void* stream, int32_t pdl);

/* ------------------------------------------------------------ sampling tail --- */

/* Device-side sampling parameters of one sequence: the layout of SamplingConfigDevice
 * (native/kernels/sm120/kernels.h:91-98), read by the kernel at run time from a fixed address so
 * that a captured step can be replayed with other values.  rep_penalty is carried for layout
 * compatibility and not applied here (the reference applies it in two kernels of its own before
 * the sampler, native/kernels/sm120/sampling.cu:293-324, on the session's token history, which is
 * not part of this path). */
typedef struct mc_sm100_sampling_config_t {
    float    temperature;       /* <= 0: the strongest candidate is returned and the generator not consumed */
    float    top_p;             /* (0, 1]; >= 1 keeps all k candidates */
    uint32_t top_k;             /* clamped to [1, 128] */
    float    rep_penalty;
    uint32_t flags, pad;
} mc_sm100_sampling_config_t;

/* Top-k / top-p / temperature sampling over bf16 logits [n_rows, vocab] (row stride in elements):
 * launch_sampling_pipeline (native/kernels/sm120/kernels.h:706-716; sampling.cu:253-531, 731-806)
 * for every row of a batch in ONE launch.  The k strongest logits under the order "value
 * descending, index ascending" (exact, ties at the threshold towards lower indices), softmax with
 * the temperature, cut at cumulative probability top_p, renormalise, draw with the xorshift64*
 * generator whose 64-bit state per row lives at d_rng_state (seed it with splitmix64(seed) as the
 * reference does, native/runtime/decode_executor.cpp:476-486; the state must not be 0).  The tail's
 * arithmetic follows the reference statement by statement.  d_cfg: [n_rows] in device memory.
 * n_rows <= 64.  No scratch memory. */
MC_SM100_API mc_status_t mc_sm100_sample_topk_topp(const uint16_t* d_logits, uint32_t n_rows, uint32_t vocab,
                                                   uint32_t row_stride, const mc_sm100_sampling_config_t* d_cfg,
                                                   uint64_t* d_rng_state, int32_t* d_out_token, void* stream,
                                                   int32_t pdl);

/* The same over vocab shards (no counterpart in the reference, which is single-GPU and samples
 * solo sessions only, docs/EXPERIMENT_LOG.md:169): every rank finds the k strongest of ITS shard
 * (d_logits holds `vocab` columns of the shard, index_base = global index of column 0), stores them
 * into every rank's exchange region through peer mappings (plain 64-bit stores, then one word per
 * (rank, row) that carries the exchange number, st.release.sys), waits -- bounded, timeout_ns, 0 =
 * 1 s, sticky through *d_status -- for all ranks' candidates, merges them with the same total order
 * and draws with ITS copy of the generator state: ranks that were seeded alike draw the same token.
 * The region (mc_sm100_sampling_exchange_bytes(max_rows, world) bytes, zeroed once, same layout on
 * every rank) is peer-mapped by the caller; d_region_peers: device array of `world` addresses as
 * mapped in this process; d_step: two device words {1, 0} at start, advanced by the kernel (the
 * exchange number, and the count of rows that have finished the current one).  A token of -1
 * means the wait ran out.  No multicast; plain peer stores and loads only. */
MC_SM100_API size_t mc_sm100_sampling_exchange_bytes(uint32_t max_rows, uint32_t world);
MC_SM100_API mc_status_t mc_sm100_sample_topk_topp_sharded(
    const uint16_t* d_logits, uint32_t n_rows, uint32_t vocab, uint32_t row_stride, int32_t index_base,
    const mc_sm100_sampling_config_t* d_cfg, uint64_t* d_rng_state, int32_t* d_out_token,
    const uint64_t* d_region_peers, const void* d_my_region, uint32_t max_rows, uint32_t* d_step,
    uint32_t rank, uint32_t world, uint64_t timeout_ns, int32_t* d_status, void* stream, int32_t pdl);

/* ------------------------------------------------- host-buffer convenience -- */

/* One linear call with HOST activations: copies h_x [M,K] to the device,
 * runs the matching kernel above on weights already resident in device
 * memory, copies y back and synchronises the stream.  kind: 0 plain linear,
 * 1 gate_up + SwiGLU epilogue (interleaved weights).  d_scale NULL = bf16
 * weights.  d_x_stage / d_y_stage are caller-provided device staging buffers
 * (M*K and M*N bf16), d_workspace as for mc_sm100_gemm_bf16.  This is the
 * call the end-to-end benchmark times; it mirrors what mc_decode_one does
 * around a step (H2D of the step input, D2H of the result, one sync;
 * native/runtime/decode_executor.cpp:163-289). */
MC_SM100_API mc_status_t mc_sm100_linear_host(int32_t kind, const void* d_w, const float* d_scale,
                                 const uint16_t* h_x, uint16_t* h_y, uint32_t M, uint32_t N,
                                 uint32_t K, uint16_t* d_x_stage, uint16_t* d_y_stage,
                                 void* d_workspace, size_t ws_size, void* stream);

/* ------------------------------------------------------------ decode stack --- */

/* The linear layers of a whole decode step as one object: weight-arena layout,
 * per-layer dispatch and CUDA-graph replay -- the part of the reference's
 * executors that belongs to this path (run_real_forward's linear dispatch,
 * native/runtime/forward.cpp:98-160, 206-237, 306-373, 443-462; mc_batch_step's GEMM
 * sequence, native/runtime/batch_group.cpp:745-807; section placement,
 * native/runtime/weight_loader.cpp:355-365, 563-630; capture and replay,
 * native/runtime/decode_executor.cpp:163-209).  Attention is stood in for by the
 * first `hidden` features of the fused qkv output.  Per layer:
 *   h = rmsnorm1(x) ; qkv = Wqkv h ; x += Wo qkv[:hidden] ; h = rmsnorm2(x) ;
 *   x += Wdown swiglu(Wgate_up h)      and finally  token = argmax(Wlm rmsnorm_f(x)). */
typedef struct mc_sm100_stack_desc_t {
    uint32_t struct_size;        /* caller sets sizeof(mc_sm100_stack_desc_t) */
    uint32_t layers, hidden, qkv_rows, inter, vocab;
    uint32_t precision;          /* 0 = bf16, 2 = e4m3 weight-only (values of mc_precision_t) */
    uint32_t max_batch;          /* 1..64 */
    float    eps;
    uint32_t enable_cuda_graph;
    uint32_t world, rank;        /* N-sharding over the GPUs of one node: world 0 or 1 = one GPU, else 2..8 */
    uint32_t reserved[2];        /* must be zero */
} mc_sm100_stack_desc_t;

typedef struct mc_sm100_stack* mc_sm100_stack_t;

/* Sections of the weight arena (each 256-byte aligned, compact, layer-major):
 * 0 qkv, 1 o, 2 gate_up (rows INTERLEAVED gate_j, up_j), 3 down, 4 norm1, 5 norm2,
 * 6..9 fp32 row scales of 0..3 (e4m3 only; gate_up scales interleaved too),
 * 10 lm_head, 11 final_norm, 12 lm_head scales (layer ignored for 10..12). */
MC_SM100_API mc_status_t mc_sm100_stack_sizes(const mc_sm100_stack_desc_t* desc, uint64_t* weight_bytes,
                                              uint64_t* scratch_bytes);
MC_SM100_API mc_status_t mc_sm100_stack_section(const mc_sm100_stack_desc_t* desc, uint32_t layer,
                                                uint32_t which, uint64_t* offset, uint64_t* bytes);

/* The caller owns both arenas (device memory, 256-byte aligned, sizes from
 * mc_sm100_stack_sizes) and fills the weight arena at the section offsets; the
 * object itself allocates no device memory. */
MC_SM100_API mc_status_t mc_sm100_stack_create(const mc_sm100_stack_desc_t* desc, void* d_weights,
                                               void* d_scratch, mc_sm100_stack_t* out);
MC_SM100_API void mc_sm100_stack_destroy(mc_sm100_stack_t stack);

/* One step on device buffers: x [M, hidden] bf16 -> greedy tokens [M]; stream-ordered,
 * no synchronisation (capturable). */
MC_SM100_API mc_status_t mc_sm100_stack_step(mc_sm100_stack_t stack, const uint16_t* d_x, uint32_t M,
                                             int32_t* d_tokens, void* stream);

/* Device pointer to the bf16 logits [M, vocab] the last step wrote (inside the scratch arena). */
MC_SM100_API const uint16_t* mc_sm100_stack_logits(mc_sm100_stack_t stack);

/* Device address of the stack's failure word (inside the scratch arena): 0 until a bounded wait
 * of any kernel of a step ran out (a tensor-core pipeline that stalled, a peer rank that is gone
 * or out of step), then 1 and sticky.  A caller that copies its results to the host anyway reads
 * this word in the same batch of copies; mc_sm100_stack_exchange_status reads it synchronously. */
MC_SM100_API const int32_t* mc_sm100_stack_status_word(mc_sm100_stack_t stack);

/* One step on HOST buffers: H2D of x, the step (a CUDA graph captured on first use
 * per batch size when enabled and `stream` is not the default stream, else eager
 * launches of the same kernels), D2H of the tokens and of the failure word, one stream
 * synchronise -- the shape of mc_decode_one / mc_batch_step around a step.  The first call
 * for a batch size on a stream runs its step eagerly and captures the graph for the calls
 * that follow.  MC_E_INTERNAL when the failure word is set (the tokens are then undefined). */
MC_SM100_API mc_status_t mc_sm100_stack_step_host(mc_sm100_stack_t stack, const uint16_t* h_x, uint32_t M,
                                                  int32_t* h_tokens, void* stream);

/* --------------------------------------------------------------- multi-GPU --- */

/* Sharded stack (desc.world > 1).  layers/hidden/qkv_rows/inter/vocab describe the WHOLE
 * model; every linear is split along its output rows (gate_up by (gate, up) pairs, lm_head by
 * vocab) with a uniform pitch of ceil(rows / world) rounded up to 8, rank r owning rows
 * [r*pitch, min(rows, (r+1)*pitch)); mc_sm100_stack_sizes / _section then describe THIS rank's
 * arena (norm weights whole).  At M = 1 outputs travel between ranks inside the GEMV kernels
 * (mc_sm100_gemv_sharded) as tagged words; at M > 1 one small kernel per linear scatters the [M, rows]
 * result into every rank's [M, width] buffer (mc_sm100_peer_allgather_rows).  Both go through an exchange region that every rank allocates in peer-mappable
 * memory (same size everywhere) and whose addresses, as mapped in this process, are bound once:
 *   mc_sm100_stack_exchange_bytes(desc, &n); allocate + map n bytes on every rank;
 *   mc_sm100_stack_bind_exchange(stack, addrs (host array [world], [rank] = own), stream);
 *   barrier across ranks; then every rank calls the same sequence of steps.
 * bind zeroes this rank's region.  mc_sm100_stack_exchange_status reads (and keeps) the
 * sticky failure word of any stack, sharded or not: 0 = every bounded wait so far was satisfied,
 * 1 = a wait ran out (a peer is gone or out of step, or a tensor-core pipeline stalled): the
 * outputs of that step are undefined; a sharded stack must be re-bound.
 * The 16-bit tags of the M = 1 exchange count M = 1 steps only (batched steps keep their own
 * counter), every tagged slot is rewritten by every M = 1 step, and the layer count is limited
 * to 4096, so a slot can only ever hold the current or the previous tag. */
MC_SM100_API mc_status_t mc_sm100_stack_exchange_bytes(const mc_sm100_stack_desc_t* desc, uint64_t* bytes);
MC_SM100_API mc_status_t mc_sm100_stack_bind_exchange(mc_sm100_stack_t stack, const uint64_t* h_peer_addrs,
                                                      uint64_t timeout_ns, void* stream);
MC_SM100_API mc_status_t mc_sm100_stack_exchange_status(mc_sm100_stack_t stack, int32_t* h_status, void* stream);

/* All-gather of an N-shard over NVLink peer memory in one small kernel (no counterpart in
 * the reference, which is single-GPU; native/include/minicpm_runtime.h:61).  Rank `rank`
 * stores its slice (shard_bytes, a multiple of 16) at offset rank * slot_bytes of EVERY
 * rank's gathered buffer (d_peer_bufs: device array of `world` device addresses, peer-mapped),
 * then publishes the exchange's epoch in every rank's flag array (d_peer_flags[p] points to
 * rank p's array of `world` uint32) and waits until its own flags (d_my_flags) show that all
 * ranks have done the same.  d_epoch is a device counter the kernel advances itself, so the
 * call can be captured and replayed.  The wait is bounded (timeout_ns, 0 = 1 s); if it runs
 * out the kernel sets *d_status = 1 and returns normally.  Plain peer stores only. */
MC_SM100_API mc_status_t mc_sm100_peer_allgather(const void* d_shard, uint32_t shard_bytes, uint32_t slot_bytes,
                                                 const uint64_t* d_peer_bufs, const uint64_t* d_peer_flags,
                                                 uint32_t* d_my_flags, uint32_t* d_epoch, uint32_t rank,
                                                 uint32_t world, uint64_t timeout_ns, int32_t* d_status,
                                                 void* stream, int32_t pdl);
/* The same for a batch: `rows` rows of row_bytes (contiguous in d_shard) land in column slot `rank` of
 * every rank's row-major buffer: row m at byte m * dst_pitch_bytes + rank * slot_bytes (batched sharded
 * linears: the gathered buffer is the [M, N] activation of the next GEMM). */
MC_SM100_API mc_status_t mc_sm100_peer_allgather_rows(const void* d_shard, uint32_t rows, uint32_t row_bytes,
                                                      uint32_t dst_pitch_bytes, uint32_t slot_bytes,
                                                      const uint64_t* d_peer_bufs, const uint64_t* d_peer_flags,
                                                      uint32_t* d_my_flags, uint32_t* d_epoch, uint32_t rank,
                                                      uint32_t world, uint64_t timeout_ns, int32_t* d_status,
                                                      void* stream, int32_t pdl);

/* Sharded M = 1 linear with the output exchange INSIDE the GEMV kernel (no counterpart in
 * the reference, which is single-GPU).  A gathered vector is an array of uint32 words, one per
 * element: bf16 bits in the low half, the low 16 bits of the exchange's sequence number in the
 * high half.  The producing kernel stores each output word straight into slot `rank` of every
 * rank's gathered vector (out_peer[p], peer-mapped, plain 32-bit stores); the consuming kernel
 * polls the words it needs -- bounded, timeout_ns, 0 = 1 s -- until every tag is the expected
 * one.  No flags, fences or atomics.  Sequence numbers are (*d_step - 1) * seq_mul + seq_add.
 * A wait that runs out sets *d_status = 1, after which all later waits give up at once. */
typedef struct mc_sm100_shard_io_t {
    uint32_t struct_size;          /* sizeof(mc_sm100_shard_io_t) */
    uint32_t world, rank;          /* world 2..8 */
    uint32_t in_tagged;            /* 1: d_x (prologue 0) / d_addend (prologue 1) is a tagged gathered vector */
    uint32_t in_seq_mul, in_seq_add;
    uint32_t out_slot;             /* slot pitch of the gathered output in words; 0 = output stays local (d_y, bf16) */
    uint32_t out_seq_mul, out_seq_add;
    uint32_t reserved;
    const uint32_t* d_step;        /* device word >= 1 */
    int32_t* d_status;
    uint64_t timeout_ns;
    uint64_t out_peer[8];
} mc_sm100_shard_io_t;

/* prologue: 0 = x is d_x; 1 = residual add + RMSNorm (d_x = residual in, d_addend may be NULL,
 * d_norm_w, d_res_out as in mc_sm100_gemv_rows_prologue).  epilogue: 0 = store, 1 = SwiGLU over
 * interleaved (gate, up) rows (N even, N/2 outputs).  d_scale NULL = bf16 weights, else e4m3.
 * d_y is used only when io->out_slot == 0.  N = rows of THIS rank's shard. */
MC_SM100_API mc_status_t mc_sm100_gemv_sharded(int32_t prologue, int32_t epilogue, const void* d_w,
                                               const float* d_scale, const uint16_t* d_x,
                                               const uint16_t* d_addend, const uint16_t* d_norm_w,
                                               uint16_t* d_res_out, uint16_t* d_y, uint32_t N, uint32_t K,
                                               float eps, const mc_sm100_shard_io_t* io, void* stream,
                                               int32_t pdl);

/* mc_sm100_lm_head_argmax_prologue over this rank's vocab shard (N rows, global index of row 0 =
 * index_base) whose addend is a tagged gathered vector (io->in_tagged = 1).  Logits and the
 * (value, index) of the shard stay local; mc_sm100_peer_argmax reduces them across ranks. */
MC_SM100_API mc_status_t mc_sm100_lm_head_argmax_sharded(
    const void* d_w, const float* d_scale, const uint16_t* d_res_in, const uint16_t* d_addend,
    const uint16_t* d_norm_w, uint16_t* d_res_out, uint16_t* d_logits, uint32_t N, uint32_t n, float eps,
    int32_t index_base, void* d_stage, int32_t* d_out_idx, float* d_out_val, const mc_sm100_shard_io_t* io,
    void* stream, int32_t pdl);

/* Greedy tokens over vocab shards in one single-CTA kernel: pushes this rank's (value, index) of each
 * of n_rows rows to every rank (d_pair_peers: device array of `world` addresses of each rank's
 * [world][n_rows] x 8-byte pair slots), signals, waits (bounded) for all ranks' pairs of step *d_step,
 * reduces every row with the reference's tie rule (lowest index, native/kernels/sm120/sampling.cu:26,
 * 80), writes tokens and values [n_rows], and finally advances *d_step. */
MC_SM100_API mc_status_t mc_sm100_peer_argmax(const float* d_val, const int32_t* d_idx, uint32_t n_rows,
                                              const uint64_t* d_pair_peers, const uint64_t* d_flag_peers,
                                              const uint64_t* d_my_pairs, const uint32_t* d_my_flags,
                                              uint32_t* d_step, uint32_t rank, uint32_t world,
                                              uint64_t timeout_ns, int32_t* d_status, int32_t* d_token,
                                              float* d_token_val, void* stream, int32_t pdl);

/* ------------------------------------------------------------ packed weights --- */

/* Reader of the reference's packed weight file (WPK v1: tools/minicpm_common.py:47-75,
 * 318-348) and loader into this library's arena layout; stands for
 * WeightLoader::load_wpk / load_wpk_fp8 (native/runtime/weight_loader.cpp:195-726) on
 * this path.  Files packed for target_sm 120 are accepted as they are. */
typedef struct mc_sm100_wpk* mc_sm100_wpk_t;
typedef struct mc_sm100_wpk_section_t {
    uint64_t name_hash;          /* FNV-1a 64 of the section name */
    uint32_t dtype, layout, rank;/* dtype 0 = bf16, 2 = e4m3 + fp32 row scales */
    uint32_t dims[8];
    uint64_t data_offset, data_bytes, scale_offset, scale_bytes;
} mc_sm100_wpk_section_t;

MC_SM100_API uint64_t mc_sm100_wpk_name_hash(const char* name);
/* Opens and validates header and TOC (MC_E_IO / MC_E_MODEL_MISMATCH with a message). */
MC_SM100_API mc_status_t mc_sm100_wpk_open(const char* path, mc_sm100_wpk_t* out);
MC_SM100_API void mc_sm100_wpk_close(mc_sm100_wpk_t wpk);
MC_SM100_API uint32_t mc_sm100_wpk_section_count(mc_sm100_wpk_t wpk);
MC_SM100_API mc_status_t mc_sm100_wpk_find(mc_sm100_wpk_t wpk, const char* name, mc_sm100_wpk_section_t* out);
/* Uploads rows [row_lo, row_hi) of a section (an N-shard) to device memory; with
 * interleave != 0 the section is a fused gate|up tensor, the range counts (gate_j, up_j)
 * pairs and the rows arrive interleaved (the layout mc_sm100_gate_up_swiglu reads).
 * e4m3 sections also deliver their row scales to d_scale.  Synchronous (load time). */
MC_SM100_API mc_status_t mc_sm100_wpk_upload(mc_sm100_wpk_t wpk, const char* name, uint32_t row_lo,
                                             uint32_t row_hi, int32_t interleave, void* d_data,
                                             uint64_t data_capacity, float* d_scale, void* stream);

/* Writer of the same container and the packer's e4m3 quantiser, on the host (role of the writer in
 * tools/minicpm_common.py:318-348 and of tools/quantize.py:85-113).  Files it writes are loadable by
 * the reference (target_sm 120) and by mc_sm100_wpk_open.  max_sections reserves the table of
 * contents: data starts at align256(64 + 132 * max_sections); sections are streamed to the file as
 * they are added (data 256-byte aligned, e4m3 sections carry their fp32 row scales directly behind
 * the codes), finish writes header and table and closes the file. */
typedef struct mc_sm100_wpk_writer* mc_sm100_wpk_writer_t;
MC_SM100_API mc_status_t mc_sm100_wpk_writer_create(const char* path, uint32_t max_sections, uint32_t target_sm,
                                                    const uint8_t* model_hash32, mc_sm100_wpk_writer_t* out);
/* dtype 0: h_data = bf16 bits, h_scales NULL; dtype 2: h_data = e4m3 codes, h_scales = fp32 [dims[0]]. */
MC_SM100_API mc_status_t mc_sm100_wpk_writer_add(mc_sm100_wpk_writer_t writer, const char* name, uint32_t dtype,
                                                 uint32_t rank, const uint32_t* dims, const void* h_data,
                                                 const float* h_scales);
MC_SM100_API mc_status_t mc_sm100_wpk_writer_finish(mc_sm100_wpk_writer_t writer);   /* also frees the writer */
MC_SM100_API void mc_sm100_wpk_writer_abort(mc_sm100_wpk_writer_t writer);           /* closes, deletes the file */
/* bf16 weight [N,K] -> e4m3 codes + fp32 row scales with the packer's rule: scale = max|row| / 448
 * floored at 1e-12, q = e4m3_rne_saturating(w / scale) (tools/minicpm_common.py:130-171, 204-212). */
MC_SM100_API mc_status_t mc_sm100_quantize_rows_host(const uint16_t* h_w, uint32_t N, uint32_t K, uint8_t* h_q,
                                                     float* h_scale);
/* The encoder alone: n floats -> n e4m3 codes (round to nearest even, saturating, never 0x7F / 0xFF). */
MC_SM100_API mc_status_t mc_sm100_e4m3_from_f32_host(const float* h_in, uint64_t n, uint8_t* h_out);

/* ---------------------------------------------------------------- debug hook -- */

/* Not part of the frozen surface (same standing as the reference's
 * mc_debug_* exports, native/runtime/session.cpp:631-723): selects the
 * arithmetic form of the streaming kernels per weight type for A/B runs.
 * 0 = widen to fp32 then FFMA, 1 = mixed-precision FMA on bf16 operands (both
 * in the generic M <= 4 kernel), 2 = the decode-chain M = 1 kernel (default);
 * any other value keeps the current form.  Forms 0 and 1 give identical bits;
 * form 2 sums in a different order (same contract, same tolerance). */
MC_SM100_API void mc_sm100_debug_set_math(int32_t bf16_math, int32_t fp8_math);

/* A/B hook for the L2 prefetch (process-wide): mode 0 = off, 1 = bulk prefetch, 2 = one
 * prefetch per 128-byte line; chunk_bytes = bytes per bulk instruction; evict_first != 0 marks
 * the streaming kernels' demand loads evict-first in L2; cap_bytes = most bytes per hint.
 * A negative value (0 for cap_bytes) keeps the current setting. */
MC_SM100_API void mc_sm100_debug_set_prefetch(int32_t mode, int32_t chunk_bytes, int32_t evict_first,
                                              int64_t cap_bytes);

/* A/B hook (process-wide): bf16 batched linears with at most max_m rows (default 8, at most 16; 0 = none) whose
 * weight has at most 16 rows per SM run on the register-streaming mma.sync kernel (csrc/gemm_mma_rows.cu), the
 * others on the tcgen05 kernel. */
MC_SM100_API void mc_sm100_debug_set_mma_rows(int32_t max_m);

/* Host-only views of two launch plans, for tests of the host logic (no CUDA call).  mma_rows_plan: how the
 * register-streaming GEMM cuts a weight of N rows on a device with `sms` SMs (0 = 148): block height (16 or 8 rows),
 * blocks a CTA holds at a time, rows the fullest SM walks through.  chain_plan: ring slot size of the persistent M = 1
 * kernel for a stack of these dimensions (0 = does not fit: per-linear kernels) and rows per slot for the K = hidden
 * linears, the gate_up pairs and the down projection. */
MC_SM100_API void mc_sm100_debug_mma_rows_plan(uint32_t N, uint32_t sms, uint32_t* rows, uint32_t* blocks_at_a_time, uint32_t* worst_rows);
MC_SM100_API void mc_sm100_debug_chain_plan(int32_t fp8, uint32_t hidden, uint32_t inter, uint32_t* slot_bytes, uint32_t* rows_hidden,
                                            uint32_t* rows_gate_up, uint32_t* rows_down);

/* Host-only self-test of the per-device bookkeeping behind the kernels' shared-memory opt-in (one entry per
 * device, raised once per device and size, safe under racing host threads); makes no CUDA call.  0 = passed. */
MC_SM100_API int32_t mc_sm100_debug_optin_selftest(void);

/* A/B hook (process-wide): on != 0 runs an M = 1 step of a one-GPU stack as ONE persistent kernel
 * (every linear of every layer and the lm_head; weights streamed through a shared-memory ring that
 * does not stop at the dependencies between linears; outputs handed from CTA to CTA as tagged words
 * behind one arrival counter per linear); 0 (default: it measured faster) launches one kernel per
 * linear.  Both give the same bits.  Takes effect for steps issued (and graphs captured) afterwards. */
MC_SM100_API void mc_sm100_debug_set_chain(int32_t on);

/* Every wait inside the tensor-core kernel is bounded; a wait that runs out
 * makes the kernel skip its stores and raise a device-side flag.  This reads
 * the flag (synchronising copy) and clears it: 0 = no wait ever ran out. */
MC_SM100_API int32_t mc_sm100_debug_take_error(void);

#ifdef __cplusplus
}
#endif
#endif /* MC_SM100A_LINEAR_H */
