/* mc_sm100a_runtime.h -- the linear-layer path behind entry points shaped like the
 * reference's public C ABI (native/include/minicpm_runtime.h:94-199).
 *
 * The reference's Rust host and its Prefill / Decode / BatchGroup executors reach the
 * linear layers through fourteen frozen mc_* functions.  The functions below have the same
 * shapes, argument order, ownership rules and error behaviour, one for one, and run the
 * linear slice of a decode step on B200 through mc_sm100a_linear.h: token -> embedding row
 * -> the decode stack (per layer: rmsnorm, fused qkv, o, rmsnorm, fused gate_up + SwiGLU,
 * down; then final norm, lm_head, greedy argmax) -> next token.  Attention, RoPE and the KV
 * cache are not part of this path (the attention block is stood in for by the first
 * `hidden` features of the fused qkv output), so a "sequence" here is a position counter
 * and the pre-decided next token.
 *
 * Conventions, as in the reference (minicpm_runtime.h:1-12, native/runtime/model.cpp:40-67,
 * native/runtime/error.cpp):
 *   - extern "C", fixed-width integers, POD structs whose first field is struct_size
 *     (checked at call time; abi_version too where present); reserved fields must be zero;
 *   - handles are 8-byte structs passed BY VALUE that wrap one pointer
 *     (native/runtime/internal_state.h:40-57); an out-handle is nulled on entry and stays
 *     null on failure; destroy functions accept a null handle;
 *   - every call clears the thread-local error text, returns mc_status_t, leaves an English
 *     message readable through mc_sm100_last_error() on failure, and lets no C++ exception
 *     out (anything unexpected becomes MC_E_INTERNAL);
 *   - a model is immutable and shareable after load; a session or a batch group is used by
 *     one thread at a time; a session inside a group must not be used solo nor destroyed
 *     (minicpm_runtime.h:135-148).
 * What differs from the reference, all additive: batch groups take up to 64 slots
 * (native/runtime/batch_group.cpp:52 caps at 8); the device gate wants compute capability
 * 10.x (model.cpp:133-139 wants 12.0); a directory without model.wpk gives a synthetic model
 * whose dimensions come from the options (the reference's mock model has fixed dimensions).
 */
#ifndef MC_SM100A_RUNTIME_H
#define MC_SM100A_RUNTIME_H

#include "mc_sm100a_linear.h"

#ifdef __cplusplus
extern "C" {
#endif

#define MC_SM100_ABI_VERSION 0x00020000u   /* value of MC_ABI_VERSION, minicpm_runtime.h:30 */

typedef struct mc_sm100_model { struct mc_sm100_model_impl* impl; } mc_sm100_model_t;
typedef struct mc_sm100_session { struct mc_sm100_session_impl* impl; } mc_sm100_session_t;
typedef struct mc_sm100_batch_group { struct mc_sm100_batch_group_impl* impl; } mc_sm100_batch_group_t;

/* Stands for mc_model_options_t (minicpm_runtime.h:59-69).  sizeof == 72. */
typedef struct mc_sm100_model_options_t {
    uint32_t struct_size;        /* caller sets sizeof(mc_sm100_model_options_t) */
    uint32_t abi_version;        /* caller sets MC_SM100_ABI_VERSION */
    int32_t  device_id;
    uint32_t max_sessions;       /* 1..64 */
    uint32_t precision;          /* 0 = bf16, 2 = e4m3 weight-only (values of mc_precision_t) */
    uint32_t enable_cuda_graph;
    /* a directory without model.wpk gives a synthetic model of these dimensions: weights
     * N(0, 0.02), norm weights 1 + 0.1 N(0,1), embedding N(0,1), from synth_seed */
    uint32_t synth_layers, synth_hidden, synth_qkv_rows, synth_inter, synth_vocab;
    uint32_t reserved0;          /* must be zero */
    uint64_t synth_seed;
    uint32_t reserved[4];        /* must be zero */
} mc_sm100_model_options_t;

/* Same layout as mc_generation_config_t (minicpm_runtime.h:72-80).  sizeof == 32. */
typedef struct mc_sm100_generation_config_t {
    uint32_t struct_size;
    uint32_t max_new_tokens;
    float    temperature;
    float    top_p;
    uint32_t top_k;
    float    repetition_penalty;
    uint64_t seed;
} mc_sm100_generation_config_t;

/* Same layout as mc_runtime_stats_t (minicpm_runtime.h:82-89). */
typedef struct mc_sm100_runtime_stats_t {
    uint64_t prompt_tokens;
    uint64_t generated_tokens;
    uint64_t prefill_us;
    uint64_t decode_us;
    uint64_t peak_vram_bytes;
    uint64_t cuda_graph_launches;
} mc_sm100_runtime_stats_t;

/* Same layout as mc_batch_options_t (minicpm_runtime.h:154-160).  sizeof == 32.
 * max_slots 1..64; max_context_tokens is carried for layout compatibility and ignored
 * (no KV cache on this path). */
typedef struct mc_sm100_batch_options_t {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t max_slots;
    uint32_t max_context_tokens;
    uint32_t reserved[4];        /* must be zero */
} mc_sm100_batch_options_t;

/* ---- lifecycle: mc_model_load / mc_model_destroy / mc_session_* (minicpm_runtime.h:94-112) ---- */

/* model_dir: UTF-8 directory.  With <model_dir>/model.wpk (the reference's packed weight
 * file, bf16 or e4m3 sections as options->precision says) the dimensions are read from the
 * sections `embedding`, `layer0.qkv`, `layer0.gate_up` and the layer count from the file, the
 * sections are uploaded into the decode stack's arena layout (gate_up interleaved), and the
 * model is the file's.  Without it the model is synthetic (see the options).  A directory
 * that does not exist is MC_E_IO.  Device memory is allocated here and nowhere later. */
MC_SM100_API mc_status_t mc_sm100_model_load(const char* model_dir, const mc_sm100_model_options_t* options,
                                             mc_sm100_model_t* out_model);
MC_SM100_API void mc_sm100_model_destroy(mc_sm100_model_t model);

MC_SM100_API mc_status_t mc_sm100_session_create(mc_sm100_model_t model, mc_sm100_session_t* out_session);
/* Keeps every allocation, stream and captured graph; clears the sequence state. */
MC_SM100_API mc_status_t mc_sm100_session_reset(mc_sm100_session_t session);
MC_SM100_API void mc_sm100_session_destroy(mc_sm100_session_t session);

/* ---- inference: mc_prefill / mc_decode_one (minicpm_runtime.h:116-128) ---- */

/* Host token ids in [0, vocab).  On this path the prompt only fixes the position counter and
 * the first decision: one step on the last prompt token pre-decides the next token. */
MC_SM100_API mc_status_t mc_sm100_prefill(mc_sm100_session_t session, const int32_t* token_ids, uint32_t token_count);

/* One decode step with the reference's hand-out rule (native/runtime/decode_executor.cpp:163-289):
 * *out_token is the token decided by the PREVIOUS step (the first call returns prefill's
 * decision); this call embeds it, runs the linear stack and decides the next one, which stays
 * in a fixed device buffer.  H2D none, D2H one token, one stream synchronise.  Greedy only:
 * temperature > 0 with top_k != 1 is MC_E_UNSUPPORTED on this entry point (sampling over a
 * candidate cut is mc_sm100_sample_topk_topp in mc_sm100a_linear.h). */
MC_SM100_API mc_status_t mc_sm100_decode_one(mc_sm100_session_t session, const mc_sm100_generation_config_t* config,
                                             int32_t* out_token);

MC_SM100_API mc_status_t mc_sm100_get_stats(mc_sm100_session_t session, mc_sm100_runtime_stats_t* out_stats);

/* ---- batched decode: mc_batch_group_* / mc_batch_step (minicpm_runtime.h:162-199) ---- */

/* A group owns one stream and one activation arena for max_slots rows
 * (native/runtime/batch_group.cpp:216-251, 297-341). */
MC_SM100_API mc_status_t mc_sm100_batch_group_create(mc_sm100_model_t model, const mc_sm100_batch_options_t* options,
                                                     mc_sm100_batch_group_t* out_group);
/* Takes a free slot.  MC_E_UNSUPPORTED: the session belongs to another model, the group is
 * full, or the session is already in a group.  Work the session queued earlier on its own
 * stream is ordered before the group's next step (event chain, batch_group.cpp:540-552). */
MC_SM100_API mc_status_t mc_sm100_batch_group_add(mc_sm100_batch_group_t group, mc_sm100_session_t session,
                                                  uint32_t* slot_id);
/* Between two steps.  The group's work is ordered before the session's next solo call. */
MC_SM100_API mc_status_t mc_sm100_batch_group_remove(mc_sm100_batch_group_t group, uint32_t slot_id);
/* One step for the members slot_ids[0..n) (no duplicates): hands out each member's previous
 * decision in out_tokens[i], embeds them as the n rows of one batched step (M = n through the
 * skinny GEMM path), decides and stores every member's next token.  The launch sequence of
 * each batch size is captured into a CUDA graph on first use when the model was loaded with
 * enable_cuda_graph (the per-slot token addresses live in a device table at a fixed address
 * that a small H2D refreshes, batch_group.cpp:688-716).  Greedy only, like the reference's
 * (batch_group.cpp:655-662). */
MC_SM100_API mc_status_t mc_sm100_batch_step(mc_sm100_batch_group_t group, const uint32_t* slot_ids, uint32_t n,
                                             const mc_sm100_generation_config_t* cfgs, int32_t* out_tokens);
/* Members still in the group go through the remove ordering first.  Null-safe. */
MC_SM100_API void mc_sm100_batch_group_destroy(mc_sm100_batch_group_t group);

/* ---- debug hooks (not part of the frozen surface; the reference has mc_debug_* likewise,
 * native/runtime/batch_group.cpp:866-955) ---- */

/* steps run, accumulated microseconds, members currently in the group, graphs captured */
MC_SM100_API mc_status_t mc_sm100_debug_batch_group_stats(mc_sm100_batch_group_t group, uint64_t* steps, uint64_t* decode_us,
                                                          uint32_t* members, uint32_t* graphs);
/* dimensions of a loaded model (any pointer may be NULL) */
MC_SM100_API mc_status_t mc_sm100_debug_model_dims(mc_sm100_model_t model, uint32_t* layers, uint32_t* hidden,
                                                   uint32_t* qkv_rows, uint32_t* inter, uint32_t* vocab);
/* copies the bf16 logits [vocab] of a session's last step to the host (synchronises its stream) */
MC_SM100_API mc_status_t mc_sm100_debug_session_logits(mc_sm100_session_t session, uint16_t* h_logits, uint32_t count);

#ifdef __cplusplus
}
#endif
#endif /* MC_SM100A_RUNTIME_H */
