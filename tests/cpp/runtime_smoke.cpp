// runtime_smoke.cpp -- the model / session / batch-group entry points from a plain C++ host,
// on a synthetic model (a model directory without model.wpk), patterned on the reference's
// native/tests/abi_smoke.cpp: argument validation first (NULL handles, wrong struct_size, wrong
// abi_version, non-zero reserved fields, out-handles nulled on failure), then the life cycle
// (load, session, prefill, decode_one, stats, reset reproduces the same tokens), then batch
// groups (add / remove between steps, duplicate and empty slots rejected, up to 64 slots, a batched
// step hands out the same tokens as the members' solo steps would).  No Python, no torch.
// Exit code 0 and "RUNTIME-SMOKE-OK" = every check passed.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <sys/stat.h>

#include "mc_sm100a_runtime.h"

#define REQUIRE(cond)                                                                                   \
    do {                                                                                                \
        if (!(cond)) {                                                                                  \
            std::printf("FAILED line %d: %s   (last error: %s)\n", __LINE__, #cond, mc_sm100_last_error()); \
            return 1;                                                                                   \
        }                                                                                               \
    } while (0)

static mc_sm100_model_options_t base_options(uint32_t precision) {
    mc_sm100_model_options_t o;
    std::memset(&o, 0, sizeof(o));
    o.struct_size = sizeof(o);
    o.abi_version = MC_SM100_ABI_VERSION;
    o.device_id = 0;
    o.max_sessions = 64;
    o.precision = precision;
    o.enable_cuda_graph = 1;
    o.synth_layers = 2; o.synth_hidden = 256; o.synth_qkv_rows = 384; o.synth_inter = 512; o.synth_vocab = 1000;
    o.synth_seed = 20260908;
    return o;
}

static mc_sm100_generation_config_t greedy() {
    mc_sm100_generation_config_t g;
    std::memset(&g, 0, sizeof(g));
    g.struct_size = sizeof(g);
    g.max_new_tokens = 32;
    g.top_k = 1;
    g.repetition_penalty = 1.0f;
    return g;
}

static int validation(const char* dir) {
    mc_sm100_model_t m{(mc_sm100_model_impl*)0x1};
    mc_sm100_model_options_t o = base_options(0);
    REQUIRE(mc_sm100_model_load(dir, nullptr, &m) == MC_E_INVALID_ARGUMENT);
    REQUIRE(m.impl == nullptr);                              // nulled on entry, stays null on failure
    REQUIRE(mc_sm100_model_load(nullptr, &o, &m) == MC_E_INVALID_ARGUMENT);
    REQUIRE(mc_sm100_model_load(dir, &o, nullptr) == MC_E_INVALID_ARGUMENT);
    { mc_sm100_model_options_t b = o; b.struct_size = 40; REQUIRE(mc_sm100_model_load(dir, &b, &m) == MC_E_INVALID_ARGUMENT);
      REQUIRE(std::strstr(mc_sm100_last_error(), "struct_size") != nullptr); }
    { mc_sm100_model_options_t b = o; b.abi_version = 0x00010000u; REQUIRE(mc_sm100_model_load(dir, &b, &m) == MC_E_INVALID_ARGUMENT); }
    { mc_sm100_model_options_t b = o; b.reserved[2] = 7; REQUIRE(mc_sm100_model_load(dir, &b, &m) == MC_E_INVALID_ARGUMENT); }
    { mc_sm100_model_options_t b = o; b.precision = 3; REQUIRE(mc_sm100_model_load(dir, &b, &m) == MC_E_UNSUPPORTED); }
    { mc_sm100_model_options_t b = o; b.synth_hidden = 250; REQUIRE(mc_sm100_model_load(dir, &b, &m) == MC_E_INVALID_ARGUMENT); }
    REQUIRE(mc_sm100_model_load("/nonexistent/dir/for/mc_sm100", &o, &m) == MC_E_IO);
    REQUIRE(m.impl == nullptr);

    REQUIRE(mc_sm100_model_load(dir, &o, &m) == MC_OK);
    REQUIRE(m.impl != nullptr);
    uint32_t L = 0, H = 0, Q = 0, I = 0, V = 0;
    REQUIRE(mc_sm100_debug_model_dims(m, &L, &H, &Q, &I, &V) == MC_OK && L == 2 && H == 256 && Q == 384 && I == 512 && V == 1000);

    mc_sm100_session_t s{(mc_sm100_session_impl*)0x1};
    REQUIRE(mc_sm100_session_create(mc_sm100_model_t{nullptr}, &s) == MC_E_INVALID_ARGUMENT);
    REQUIRE(s.impl == nullptr);
    REQUIRE(mc_sm100_session_create(m, nullptr) == MC_E_INVALID_ARGUMENT);
    REQUIRE(mc_sm100_session_create(m, &s) == MC_OK);

    int32_t tok = -1;
    mc_sm100_generation_config_t g = greedy();
    REQUIRE(mc_sm100_decode_one(s, nullptr, &tok) == MC_E_INVALID_ARGUMENT);
    REQUIRE(mc_sm100_decode_one(s, &g, nullptr) == MC_E_INVALID_ARGUMENT);
    { mc_sm100_generation_config_t b = g; b.struct_size = 8; REQUIRE(mc_sm100_decode_one(s, &b, &tok) == MC_E_INVALID_ARGUMENT); }
    REQUIRE(mc_sm100_decode_one(s, &g, &tok) == MC_E_INVALID_ARGUMENT);         // empty sequence: prefill first
    { mc_sm100_generation_config_t b = g; b.temperature = 0.8f; b.top_k = 40;   // not greedy
      const int32_t p3[3] = {1, 2, 3};
      REQUIRE(mc_sm100_prefill(s, p3, 3) == MC_OK);
      REQUIRE(mc_sm100_decode_one(s, &b, &tok) == MC_E_UNSUPPORTED);
      REQUIRE(mc_sm100_session_reset(s) == MC_OK); }
    const int32_t ok3[3] = {5, 17, 999}, oob[2] = {3, 1000};
    REQUIRE(mc_sm100_prefill(s, nullptr, 3) == MC_E_INVALID_ARGUMENT);
    REQUIRE(mc_sm100_prefill(s, ok3, 0) == MC_E_INVALID_ARGUMENT);
    REQUIRE(mc_sm100_prefill(s, oob, 2) == MC_E_INVALID_ARGUMENT);
    REQUIRE(mc_sm100_prefill(mc_sm100_session_t{nullptr}, ok3, 3) == MC_E_INVALID_ARGUMENT);
    mc_sm100_runtime_stats_t st;
    REQUIRE(mc_sm100_get_stats(mc_sm100_session_t{nullptr}, &st) == MC_E_INVALID_ARGUMENT);
    REQUIRE(mc_sm100_get_stats(s, nullptr) == MC_E_INVALID_ARGUMENT);
    REQUIRE(mc_sm100_prefill(s, ok3, 3) == MC_OK);
    REQUIRE(mc_sm100_decode_one(s, &g, &tok) == MC_OK);
    REQUIRE(tok >= 0 && tok < 1000);

    // max_sessions is enforced
    { mc_sm100_model_options_t one = o; one.max_sessions = 1;
      mc_sm100_model_t m1{nullptr};
      REQUIRE(mc_sm100_model_load(dir, &one, &m1) == MC_OK);
      mc_sm100_session_t a{nullptr}, b{nullptr};
      REQUIRE(mc_sm100_session_create(m1, &a) == MC_OK);
      REQUIRE(mc_sm100_session_create(m1, &b) != MC_OK && b.impl == nullptr);
      mc_sm100_session_destroy(a);
      REQUIRE(mc_sm100_session_create(m1, &b) == MC_OK);     // the slot came back
      mc_sm100_session_destroy(b);
      mc_sm100_model_destroy(m1); }

    mc_sm100_session_destroy(s);
    mc_sm100_model_destroy(m);
    return 0;
}

// solo life cycle: deterministic, reset reproduces, stats count
static int lifecycle(const char* dir, uint32_t precision, std::vector<int32_t>* tokens_out) {
    mc_sm100_model_options_t o = base_options(precision);
    mc_sm100_model_t m{nullptr};
    REQUIRE(mc_sm100_model_load(dir, &o, &m) == MC_OK);
    mc_sm100_session_t s{nullptr};
    REQUIRE(mc_sm100_session_create(m, &s) == MC_OK);
    const int32_t prompt[3] = {11, 22, 33};
    mc_sm100_generation_config_t g = greedy();
    std::vector<int32_t> first, second;
    REQUIRE(mc_sm100_prefill(s, prompt, 3) == MC_OK);
    for (int i = 0; i < 12; ++i) {
        int32_t tok = -1;
        REQUIRE(mc_sm100_decode_one(s, &g, &tok) == MC_OK);
        REQUIRE(tok >= 0 && tok < 1000);
        first.push_back(tok);
    }
    mc_sm100_runtime_stats_t st;
    REQUIRE(mc_sm100_get_stats(s, &st) == MC_OK);
    REQUIRE(st.prompt_tokens == 3 && st.generated_tokens == 12 && st.decode_us > 0 && st.peak_vram_bytes > 0);
    REQUIRE(st.cuda_graph_launches >= 10);                  // eager first, captured graph afterwards
    REQUIRE(mc_sm100_session_reset(s) == MC_OK);
    REQUIRE(mc_sm100_get_stats(s, &st) == MC_OK && st.generated_tokens == 0);
    REQUIRE(mc_sm100_prefill(s, prompt, 3) == MC_OK);
    for (int i = 0; i < 12; ++i) {
        int32_t tok = -1;
        REQUIRE(mc_sm100_decode_one(s, &g, &tok) == MC_OK);
        second.push_back(tok);
    }
    REQUIRE(first == second);                                // same prompt, greedy: same tokens (graph replay == eager)
    bool varied = false;
    for (size_t i = 1; i < first.size(); ++i) varied = varied || first[i] != first[0];
    REQUIRE(varied);                                         // the chain really maps token -> next token
    if (tokens_out) *tokens_out = first;
    mc_sm100_session_destroy(s);
    mc_sm100_model_destroy(m);
    return 0;
}

static int batch(const char* dir, uint32_t precision) {
    mc_sm100_model_options_t o = base_options(precision);
    mc_sm100_model_t m{nullptr}, other{nullptr};
    REQUIRE(mc_sm100_model_load(dir, &o, &m) == MC_OK);
    REQUIRE(mc_sm100_model_load(dir, &o, &other) == MC_OK);

    mc_sm100_batch_options_t bo;
    std::memset(&bo, 0, sizeof(bo));
    bo.struct_size = sizeof(bo); bo.abi_version = MC_SM100_ABI_VERSION; bo.max_slots = 64; bo.max_context_tokens = 4096;
    mc_sm100_batch_group_t g{(mc_sm100_batch_group_impl*)0x1};
    REQUIRE(mc_sm100_batch_group_create(mc_sm100_model_t{nullptr}, &bo, &g) == MC_E_INVALID_ARGUMENT);
    REQUIRE(g.impl == nullptr);
    REQUIRE(mc_sm100_batch_group_create(m, nullptr, &g) == MC_E_INVALID_ARGUMENT);
    { mc_sm100_batch_options_t b = bo; b.struct_size = 16; REQUIRE(mc_sm100_batch_group_create(m, &b, &g) == MC_E_INVALID_ARGUMENT); }
    { mc_sm100_batch_options_t b = bo; b.abi_version = 1; REQUIRE(mc_sm100_batch_group_create(m, &b, &g) == MC_E_INVALID_ARGUMENT); }
    { mc_sm100_batch_options_t b = bo; b.reserved[1] = 1; REQUIRE(mc_sm100_batch_group_create(m, &b, &g) == MC_E_INVALID_ARGUMENT); }
    { mc_sm100_batch_options_t b = bo; b.max_slots = 65; REQUIRE(mc_sm100_batch_group_create(m, &b, &g) == MC_E_UNSUPPORTED); }
    { mc_sm100_batch_options_t b = bo; b.max_slots = 0; REQUIRE(mc_sm100_batch_group_create(m, &b, &g) == MC_E_UNSUPPORTED); }
    REQUIRE(mc_sm100_batch_group_create(m, &bo, &g) == MC_OK);      // 64 slots: the reference stops at 8

    // solo reference runs: member i starts from prompt {i+1} and decodes 6 tokens on its own
    const uint32_t NS = 20, STEPS = 6;
    mc_sm100_generation_config_t gc = greedy();
    std::vector<std::vector<int32_t>> solo(NS);
    std::vector<mc_sm100_session_t> ss(NS);
    for (uint32_t i = 0; i < NS; ++i) {
        ss[i] = mc_sm100_session_t{nullptr};
        REQUIRE(mc_sm100_session_create(m, &ss[i]) == MC_OK);
        const int32_t p = (int32_t)(i * 37 + 1);
        REQUIRE(mc_sm100_prefill(ss[i], &p, 1) == MC_OK);
        for (uint32_t t = 0; t < STEPS; ++t) {
            int32_t tok = -1;
            REQUIRE(mc_sm100_decode_one(ss[i], &gc, &tok) == MC_OK);
            solo[i].push_back(tok);
        }
        REQUIRE(mc_sm100_session_reset(ss[i]) == MC_OK);
        REQUIRE(mc_sm100_prefill(ss[i], &p, 1) == MC_OK);
    }
    // membership rules
    uint32_t slot = 99;
    mc_sm100_session_t foreign{nullptr};
    REQUIRE(mc_sm100_session_create(other, &foreign) == MC_OK);
    REQUIRE(mc_sm100_batch_group_add(g, foreign, &slot) == MC_E_UNSUPPORTED);          // another model
    REQUIRE(mc_sm100_batch_group_add(mc_sm100_batch_group_t{nullptr}, ss[0], &slot) == MC_E_INVALID_ARGUMENT);
    REQUIRE(mc_sm100_batch_group_add(g, ss[0], nullptr) == MC_E_INVALID_ARGUMENT);
    std::vector<uint32_t> slots(NS);
    for (uint32_t i = 0; i < NS; ++i) REQUIRE(mc_sm100_batch_group_add(g, ss[i], &slots[i]) == MC_OK && slots[i] == i);
    REQUIRE(mc_sm100_batch_group_add(g, ss[3], &slot) == MC_E_UNSUPPORTED);            // already a member
    int32_t tok = -1;
    REQUIRE(mc_sm100_decode_one(ss[3], &gc, &tok) == MC_E_UNSUPPORTED);                // busy: no solo use inside a group
    REQUIRE(mc_sm100_batch_group_remove(g, 40) == MC_E_INVALID_ARGUMENT);              // empty slot

    // step validation
    std::vector<mc_sm100_generation_config_t> cfgs(64, gc);
    std::vector<int32_t> out(64, -1);
    { const uint32_t dup[2] = {1, 1}; REQUIRE(mc_sm100_batch_step(g, dup, 2, cfgs.data(), out.data()) == MC_E_INVALID_ARGUMENT); }
    { const uint32_t empty[1] = {33}; REQUIRE(mc_sm100_batch_step(g, empty, 1, cfgs.data(), out.data()) == MC_E_INVALID_ARGUMENT); }
    { const uint32_t one[1] = {0}; REQUIRE(mc_sm100_batch_step(g, one, 0, cfgs.data(), out.data()) == MC_E_INVALID_ARGUMENT);
      REQUIRE(mc_sm100_batch_step(g, nullptr, 1, cfgs.data(), out.data()) == MC_E_INVALID_ARGUMENT);
      std::vector<mc_sm100_generation_config_t> bad(1, gc); bad[0].temperature = 1.0f; bad[0].top_k = 50;
      REQUIRE(mc_sm100_batch_step(g, one, 1, bad.data(), out.data()) == MC_E_UNSUPPORTED);
      bad[0] = gc; bad[0].struct_size = 4;
      REQUIRE(mc_sm100_batch_step(g, one, 1, bad.data(), out.data()) == MC_E_INVALID_ARGUMENT); }

    // The scenario below runs twice from the same prompts; its handed-out tokens must repeat exactly
    // (eager first, captured graphs afterwards: replay == eager).  Against the solo runs: the first
    // batched step hands out the prefill decisions (exactly the solo ones); later steps hand out
    // decisions taken by the batched kernels, whose sums run in another order than the M = 1 kernel's,
    // so a near-tie between two logits may resolve differently for an occasional member.
    const uint32_t a4[4] = {0, 1, 2, 3}, a3[3] = {0, 1, 3};
    std::vector<uint32_t> b16;
    for (uint32_t i = 4; i < NS; ++i) b16.push_back(i);
    std::vector<int32_t> runs[2];
    for (int run = 0; run < 2; ++run) {
        std::vector<int32_t>& rec = runs[run];
        if (run == 1) {                                      // start over: everybody out, reset, same prompts, back in
            for (uint32_t i = 0; i < NS; ++i) REQUIRE(mc_sm100_batch_group_remove(g, i) == MC_OK);
            for (uint32_t i = 0; i < NS; ++i) {
                const int32_t p = (int32_t)(i * 37 + 1);
                REQUIRE(mc_sm100_session_reset(ss[i]) == MC_OK);
                REQUIRE(mc_sm100_prefill(ss[i], &p, 1) == MC_OK);
                REQUIRE(mc_sm100_batch_group_add(g, ss[i], &slot) == MC_OK && slot == i);
            }
        }
        uint32_t same1 = 0;
        for (uint32_t t = 0; t < 3; ++t) {
            REQUIRE(mc_sm100_batch_step(g, a4, 4, cfgs.data(), out.data()) == MC_OK);
            for (uint32_t i = 0; i < 4; ++i) {
                REQUIRE(out[i] >= 0 && out[i] < 1000);
                if (t == 0) REQUIRE(out[i] == solo[i][0]);
                if (t == 1) same1 += out[i] == solo[i][1] ? 1u : 0u;
                rec.push_back(out[i]);
            }
            REQUIRE(mc_sm100_batch_step(g, b16.data(), 16, cfgs.data(), out.data()) == MC_OK);
            for (uint32_t i = 0; i < 16; ++i) {
                REQUIRE(out[i] >= 0 && out[i] < 1000);
                if (t == 0) REQUIRE(out[i] == solo[4 + i][0]);
                if (t == 1) same1 += out[i] == solo[4 + i][1] ? 1u : 0u;
                rec.push_back(out[i]);
            }
        }
        REQUIRE(same1 >= 15);                                // of 20 members
        // a member leaves between steps, continues solo where the group left it, and comes back
        REQUIRE(mc_sm100_batch_group_remove(g, 2) == MC_OK);
        REQUIRE(mc_sm100_decode_one(ss[2], &gc, &tok) == MC_OK);
        rec.push_back(tok);
        REQUIRE(mc_sm100_batch_step(g, a3, 3, cfgs.data(), out.data()) == MC_OK);
        for (uint32_t i = 0; i < 3; ++i) rec.push_back(out[i]);
        REQUIRE(mc_sm100_batch_group_add(g, ss[2], &slot) == MC_OK && slot == 2);    // the freed slot
        REQUIRE(mc_sm100_batch_step(g, a4, 4, cfgs.data(), out.data()) == MC_OK);
        for (uint32_t i = 0; i < 4; ++i) rec.push_back(out[i]);
    }
    REQUIRE(runs[0] == runs[1]);

    uint64_t steps = 0, us = 0;
    uint32_t members = 0, graphs = 0;
    REQUIRE(mc_sm100_debug_batch_group_stats(g, &steps, &us, &members, &graphs) == MC_OK);
    REQUIRE(steps == 16 && members == NS && us > 0);
    REQUIRE(graphs == 3);                                    // one captured graph per batch size used: 4, 16, 3

    // fill all 64 slots and step once with everybody
    std::vector<mc_sm100_session_t> extra;
    for (uint32_t i = NS; i < 63; ++i) {                     // `foreign` holds a session of the other model; 63 of ours + it = limit
        mc_sm100_session_t e{nullptr};
        REQUIRE(mc_sm100_session_create(m, &e) == MC_OK);
        const int32_t p = (int32_t)(i + 100);
        REQUIRE(mc_sm100_prefill(e, &p, 1) == MC_OK);
        REQUIRE(mc_sm100_batch_group_add(g, e, &slot) == MC_OK && slot == i);
        extra.push_back(e);
    }
    std::vector<uint32_t> all;
    for (uint32_t i = 0; i < 63; ++i) all.push_back(i);
    REQUIRE(mc_sm100_batch_step(g, all.data(), 63, cfgs.data(), out.data()) == MC_OK);
    for (uint32_t i = 0; i < 63; ++i) REQUIRE(out[i] >= 0 && out[i] < 1000);

    mc_sm100_batch_group_destroy(g);                         // members leave through the remove ordering
    REQUIRE(mc_sm100_decode_one(ss[0], &gc, &tok) == MC_OK); // usable solo again
    for (auto& s : ss) mc_sm100_session_destroy(s);
    for (auto& s : extra) mc_sm100_session_destroy(s);
    mc_sm100_session_destroy(foreign);
    mc_sm100_model_destroy(other);
    mc_sm100_model_destroy(m);
    return 0;
}

int main(int argc, char** argv) {
    const std::string dir = argc > 1 ? argv[1] : "mc_sm100_smoke_model_dir";
    ::mkdir(dir.c_str(), 0755);
    // null-safe destroys
    mc_sm100_session_destroy(mc_sm100_session_t{nullptr});
    mc_sm100_model_destroy(mc_sm100_model_t{nullptr});
    mc_sm100_batch_group_destroy(mc_sm100_batch_group_t{nullptr});
    static_assert(sizeof(mc_sm100_generation_config_t) == 32 && sizeof(mc_sm100_batch_options_t) == 32 &&
                  sizeof(mc_sm100_model_options_t) == 72 && sizeof(mc_sm100_model_t) == 8 && sizeof(mc_sm100_session_t) == 8 &&
                  sizeof(mc_sm100_batch_group_t) == 8, "ABI sizes");
    if (validation(dir.c_str())) return 1;
    std::vector<int32_t> bf16_tokens, fp8_tokens;
    if (lifecycle(dir.c_str(), 0, &bf16_tokens)) return 1;
    if (lifecycle(dir.c_str(), 2, &fp8_tokens)) return 1;
    if (batch(dir.c_str(), 0)) return 1;
    if (batch(dir.c_str(), 2)) return 1;
    std::printf("RUNTIME-SMOKE-OK bf16 first tokens %d %d %d, e4m3 %d %d %d\n", bf16_tokens[0], bf16_tokens[1], bf16_tokens[2],
                fp8_tokens[0], fp8_tokens[1], fp8_tokens[2]);
    return 0;
}
