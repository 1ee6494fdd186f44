// runtime_abi.cu -- model / session / batch-group objects shaped like the reference's public
// C ABI, over the decode stack.
//
// Stands where native/runtime/model.cpp (load, options validation, device gate),
// native/runtime/session.cpp + decode_executor.cpp (prefill, decode_one with the "hand out the
// previous decision" rule, per-session graph) and native/runtime/batch_group.cpp (create / add /
// remove / step / destroy, step table at fixed device addresses, event chains between member and
// group streams) stand in the reference -- for the linear-layer slice of a step only.  Everything
// is allocated at load / create time; a step allocates nothing and makes no host decision that
// depends on device data.
#include <atomic>
#include <chrono>
#include <cstring>
#include <new>
#include <string>

#include <sys/stat.h>

#include "common.cuh"
#include "mc_sm100a_runtime.h"

namespace mcl {

constexpr uint32_t kMaxSlots = 64;

// ---- small kernels of the shim ----------------------------------------------------------------

// x[row, :] = embedding[token(row), :]; the token of a row is read through a table of device
// addresses (batch: each member's own next-token word) or from `direct` (solo).  The token that was
// read is also written to emitted[row]: it is the decision the host hands out for this step.
__global__ void embed_rows_kernel(const uint16_t* __restrict__ emb, const int32_t* const* __restrict__ tok_ptrs,
                                  const int32_t* __restrict__ direct, uint16_t* __restrict__ x, int32_t* __restrict__ emitted,
                                  uint32_t H, uint32_t V) {
    pdl_trigger();
    pdl_wait();
    const uint32_t row = blockIdx.x;
    const int32_t tok = tok_ptrs != nullptr ? *tok_ptrs[row] : direct[row];
    if (threadIdx.x == 0) emitted[row] = tok;
    const uint32_t t = (tok < 0 || (uint32_t)tok >= V) ? 0u : (uint32_t)tok;   // a bad token is reported by the host, never dereferenced
    const uint4* src = reinterpret_cast<const uint4*>(emb + (size_t)t * H);
    uint4* dst = reinterpret_cast<uint4*>(x + (size_t)row * H);
    for (uint32_t i = threadIdx.x; i < H / 8u; i += blockDim.x) dst[i] = src[i];
}

// *tok_ptrs[i] = tokens[i]: the step's decisions back into each member's own next-token word
__global__ void scatter_tokens_kernel(const int32_t* __restrict__ tokens, int32_t* const* __restrict__ tok_ptrs, uint32_t n) {
    pdl_trigger();
    pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) *tok_ptrs[i] = tokens[i];
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// p[i] = bf16(mean + std * N(0,1)), counter-based (the value of element i depends on (seed, i) only)
__global__ void fill_normal_bf16_kernel(uint16_t* __restrict__ p, size_t n, uint64_t seed, float mean, float stdv) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const uint64_t r = mix64(seed * 0xD1342543DE82EF95ull + i);
        const float u1 = ((float)(uint32_t)(r >> 40) + 1.0f) * (1.0f / 16777217.0f);    // (0, 1)
        const float u2 = (float)(uint32_t)((r >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);
        const float g = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        p[i] = f32_to_bf16_bits(mean + stdv * g);
    }
}

// bf16 rows -> e4m3 codes + fp32 row scale with the packer's rule: scale = max(max|row| / 448, 1e-12),
// q = e4m3_rne_saturating(w / scale) (tools/minicpm_common.py:204-212).  One CTA per row.
__global__ void quantize_weight_rows_kernel(const uint16_t* __restrict__ w, uint8_t* __restrict__ q, float* __restrict__ scale,
                                            uint32_t N, uint32_t K) {
    __shared__ float wmax[8];
    __shared__ float s_scale;
    for (uint32_t row = blockIdx.x; row < N; row += gridDim.x) {
        const uint16_t* wr = w + (size_t)row * K;
        float am = 0.f;
        for (uint32_t k = threadIdx.x; k < K; k += blockDim.x) am = fmaxf(am, fabsf(__uint_as_float((uint32_t)wr[k] << 16)));
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, s));
        if ((threadIdx.x & 31u) == 0u) wmax[threadIdx.x >> 5] = am;
        __syncthreads();
        if (threadIdx.x == 0) {
            float v = wmax[0];
            for (uint32_t i = 1; i < blockDim.x / 32u; ++i) v = fmaxf(v, wmax[i]);
            s_scale = fmaxf(v / 448.0f, 1e-12f);
            scale[row] = s_scale;
        }
        __syncthreads();
        const float sc = s_scale;
        for (uint32_t k = threadIdx.x; k < K; k += blockDim.x) {
            const float v = __uint_as_float((uint32_t)wr[k] << 16) / sc;
            uint16_t packed;
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(0.0f), "f"(v));
            q[(size_t)row * K + k] = (uint8_t)(packed & 0xFFu);
        }
        __syncthreads();
    }
}

}  // namespace mcl

using namespace mcl;

// ---- objects ----------------------------------------------------------------------------------

struct mc_sm100_model_impl {
    int device;
    uint32_t L, H, Q, I, V, precision, graph, max_sessions;
    uint8_t* d_weights;
    uint16_t* d_embedding;
    uint64_t weight_bytes, vram_bytes;
    std::atomic<uint32_t> sessions;
    mc_sm100_stack_desc_t desc(uint32_t max_batch) const {
        mc_sm100_stack_desc_t d{};
        d.struct_size = sizeof(d);
        d.layers = L; d.hidden = H; d.qkv_rows = Q; d.inter = I; d.vocab = V;
        d.precision = precision; d.max_batch = max_batch; d.eps = 1e-6f; d.enable_cuda_graph = 0;
        return d;
    }
};

struct mc_sm100_session_impl {
    mc_sm100_model_impl* model;
    cudaStream_t stream;
    uint8_t* d_block;              // one allocation: stack scratch | x [H] | next token | emitted token
    mc_sm100_stack_t stack;
    uint16_t* d_x;
    int32_t* d_next_token;
    int32_t* d_emitted;
    int32_t* h_word;               // pinned: [0] emitted token, [1] failure word, [2] staging of a token H2D
    cudaGraphExec_t graph;
    uint32_t seq_len;
    mc_sm100_runtime_stats_t stats;
    mc_sm100_batch_group_impl* group;   // busy marker while the session is a member
};

struct mc_sm100_batch_group_impl {
    mc_sm100_model_impl* model;
    cudaStream_t stream;
    uint32_t max_slots;
    mc_sm100_session_impl* members[kMaxSlots];
    uint8_t* d_block;              // stack scratch | x [max][H] | tokens [max] | emitted [max] | token address table [max]
    mc_sm100_stack_t stack;
    uint16_t* d_x;
    int32_t* d_tokens;
    int32_t* d_emitted;
    int32_t** d_step_tok;
    int32_t** h_step_tok;          // pinned staging of the table
    int32_t* h_words;              // pinned: [0..max) emitted tokens, [max] failure word
    cudaEvent_t ev_member[kMaxSlots], ev_group;
    cudaGraphExec_t graph[kMaxSlots + 1];
    uint64_t steps, decode_us;
    uint32_t graphs;
};

namespace {

inline size_t align256(size_t v) { return (v + 255u) & ~(size_t)255u; }

#define MC_TRY try {
#define MC_CATCH(who)                                                    \
    } catch (...) {                                                      \
        set_error("%s: internal error (uncaught exception)", who);       \
        return MC_E_INTERNAL;                                            \
    }

bool greedy_only(const mc_sm100_generation_config_t& c) { return !(c.temperature > 0.f && c.top_k != 1u); }

mc_status_t cuda_fail(const char* who, const char* what, cudaError_t e) {
    (void)cudaGetLastError();
    set_error("%s: %s failed: %s", who, what, cudaGetErrorString(e));
    return e == cudaErrorMemoryAllocation ? MC_E_OUT_OF_MEMORY : MC_E_CUDA;
}

// The launches of one step for `rows` rows; `tok_ptrs` null = solo (token read from `direct`).
mc_status_t enqueue_step(const mc_sm100_model_impl* m, mc_sm100_stack_t stack, const int32_t* const* tok_ptrs, const int32_t* direct,
                         uint16_t* d_x, int32_t* d_emitted, int32_t* d_tokens, uint32_t rows, cudaStream_t st) {
    (void)launch(embed_rows_kernel, dim3(rows), dim3(128), 0, st, true, (const uint16_t*)m->d_embedding, tok_ptrs, direct, d_x, d_emitted,
                 m->H, m->V);
    MCL_CHECK_LAUNCH("embed_rows");
    const mc_status_t rc = mc_sm100_stack_step(stack, d_x, rows, d_tokens, (void*)st);
    if (rc != MC_OK) return rc;
    if (tok_ptrs != nullptr) {
        (void)launch(scatter_tokens_kernel, dim3(1), dim3(64), 0, st, true, (const int32_t*)d_tokens, (int32_t* const*)tok_ptrs, rows);
        MCL_CHECK_LAUNCH("scatter_tokens");
    }
    return MC_OK;
}

// Captures `body` (which only enqueues on `st`) into an executable graph; leaves *out null when
// capture is not possible -- the caller then launches eagerly (native/runtime/session.cpp:489-499).
template <typename Body>
void capture_graph(cudaStream_t st, cudaGraphExec_t* out, Body body) {
    *out = nullptr;
    cudaGraph_t g = nullptr;
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { (void)cudaGetLastError(); return; }
    const mc_status_t rc = body();
    const cudaError_t ce = cudaStreamEndCapture(st, &g);
    if (rc == MC_OK && ce == cudaSuccess && g != nullptr && cudaGraphInstantiate(out, g, 0) != cudaSuccess) *out = nullptr;
    if (g != nullptr) cudaGraphDestroy(g);
    (void)cudaGetLastError();
    clear_error();
}

bool dir_exists(const char* p) { struct stat sb; return ::stat(p, &sb) == 0 && S_ISDIR(sb.st_mode); }
bool file_exists(const std::string& p) { struct stat sb; return ::stat(p.c_str(), &sb) == 0 && S_ISREG(sb.st_mode); }

void* weight_ptr(const mc_sm100_model_impl* m, const mc_sm100_stack_desc_t& d, uint32_t layer, uint32_t which, uint64_t* bytes) {
    uint64_t off = 0, n = 0;
    if (mc_sm100_stack_section(&d, layer, which, &off, &n) != MC_OK || n == 0) { if (bytes) *bytes = 0; return nullptr; }
    if (bytes) *bytes = n;
    return m->d_weights + off;
}

mc_status_t fill_synthetic(mc_sm100_model_impl* m, uint64_t seed) {
    const mc_sm100_stack_desc_t d = m->desc(1);
    const bool fp8 = m->precision == 2u;
    uint16_t* tmp = nullptr;
    if (fp8) {
        const size_t biggest = (size_t)(m->V > 2u * m->I ? m->V : 2u * m->I) * (m->H > m->I ? m->H : m->I);   // generous
        const cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&tmp), biggest * 2u);
        if (e != cudaSuccess) return cuda_fail("mc_sm100_model_load", "cudaMalloc (quantiser staging)", e);
    }
    uint64_t id = 0;
    auto matrix = [&](uint32_t layer, uint32_t wsec, uint32_t ssec, uint32_t N, uint32_t K) {
        void* w = weight_ptr(m, d, layer, wsec, nullptr);
        ++id;
        if (!fp8) {
            fill_normal_bf16_kernel<<<592, 256>>>((uint16_t*)w, (size_t)N * K, seed * 1000003ull + id, 0.f, 0.02f);
        } else {
            fill_normal_bf16_kernel<<<592, 256>>>(tmp, (size_t)N * K, seed * 1000003ull + id, 0.f, 0.02f);
            quantize_weight_rows_kernel<<<N < 4096u ? N : 4096u, 256>>>(tmp, (uint8_t*)w, (float*)weight_ptr(m, d, layer, ssec, nullptr), N, K);
        }
    };
    auto norm = [&](uint32_t layer, uint32_t sec) {
        ++id;
        fill_normal_bf16_kernel<<<8, 256>>>((uint16_t*)weight_ptr(m, d, layer, sec, nullptr), m->H, seed * 1000003ull + id, 1.0f, 0.1f);
    };
    for (uint32_t l = 0; l < m->L; ++l) {
        matrix(l, 0, 6, m->Q, m->H); matrix(l, 1, 7, m->H, m->H); matrix(l, 2, 8, 2u * m->I, m->H); matrix(l, 3, 9, m->H, m->I);
        norm(l, 4); norm(l, 5);
    }
    matrix(0, 10, 12, m->V, m->H);
    norm(0, 11);
    ++id;
    fill_normal_bf16_kernel<<<592, 256>>>(m->d_embedding, (size_t)m->V * m->H, seed * 1000003ull + id, 0.f, 1.0f);
    cudaError_t e = cudaDeviceSynchronize();
    if (tmp != nullptr) cudaFree(tmp);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail("mc_sm100_model_load", "synthetic weight fill", e);
    return MC_OK;
}

mc_status_t upload_wpk(mc_sm100_model_impl* m, mc_sm100_wpk_t wpk) {
    const mc_sm100_stack_desc_t d = m->desc(1);
    auto put = [&](const char* name, uint32_t layer, uint32_t wsec, uint32_t ssec, uint32_t rows, int interleave) -> mc_status_t {
        uint64_t bytes = 0;
        void* w = weight_ptr(m, d, layer, wsec, &bytes);
        float* sc = ssec != 0xFFu ? (float*)weight_ptr(m, d, layer, ssec, nullptr) : nullptr;
        return mc_sm100_wpk_upload(wpk, name, 0, rows, interleave, w, bytes, sc, nullptr);
    };
    char name[64];
    for (uint32_t l = 0; l < m->L; ++l) {
        mc_status_t rc;
        std::snprintf(name, sizeof(name), "layer%u.qkv", l);      if ((rc = put(name, l, 0, 6, m->Q, 0)) != MC_OK) return rc;
        std::snprintf(name, sizeof(name), "layer%u.o", l);        if ((rc = put(name, l, 1, 7, m->H, 0)) != MC_OK) return rc;
        std::snprintf(name, sizeof(name), "layer%u.gate_up", l);  if ((rc = put(name, l, 2, 8, m->I, 1)) != MC_OK) return rc;
        std::snprintf(name, sizeof(name), "layer%u.down", l);     if ((rc = put(name, l, 3, 9, m->H, 0)) != MC_OK) return rc;
        std::snprintf(name, sizeof(name), "layer%u.norm1", l);    if ((rc = put(name, l, 4, 0xFFu, m->H, 0)) != MC_OK) return rc;
        std::snprintf(name, sizeof(name), "layer%u.norm2", l);    if ((rc = put(name, l, 5, 0xFFu, m->H, 0)) != MC_OK) return rc;
    }
    mc_status_t rc = put("lm_head", 0, 10, 12, m->V, 0);
    if (rc == MC_OK) rc = put("final_norm", 0, 11, 0xFFu, m->H, 0);
    if (rc == MC_OK) rc = mc_sm100_wpk_upload(wpk, "embedding", 0, m->V, 0, m->d_embedding, (uint64_t)m->V * m->H * 2u, nullptr, nullptr);
    return rc;
}

void release_model(mc_sm100_model_impl* m) {
    if (m == nullptr) return;
    if (m->d_weights != nullptr) cudaFree(m->d_weights);
    if (m->d_embedding != nullptr) cudaFree(m->d_embedding);
    delete m;
}

void release_session(mc_sm100_session_impl* s) {
    if (s == nullptr) return;
    if (s->stream != nullptr) (void)cudaStreamSynchronize(s->stream);
    if (s->graph != nullptr) cudaGraphExecDestroy(s->graph);
    if (s->stack != nullptr) mc_sm100_stack_destroy(s->stack);
    if (s->d_block != nullptr) cudaFree(s->d_block);
    if (s->h_word != nullptr) cudaFreeHost(s->h_word);
    if (s->stream != nullptr) cudaStreamDestroy(s->stream);
    if (s->model != nullptr) s->model->sessions.fetch_sub(1);
    delete s;
}

void release_group(mc_sm100_batch_group_impl* g) {
    if (g == nullptr) return;
    if (g->stream != nullptr) (void)cudaStreamSynchronize(g->stream);
    for (auto& e : g->graph) if (e != nullptr) cudaGraphExecDestroy(e);
    for (auto& e : g->ev_member) if (e != nullptr) cudaEventDestroy(e);
    if (g->ev_group != nullptr) cudaEventDestroy(g->ev_group);
    if (g->stack != nullptr) mc_sm100_stack_destroy(g->stack);
    if (g->d_block != nullptr) cudaFree(g->d_block);
    if (g->h_step_tok != nullptr) cudaFreeHost(g->h_step_tok);
    if (g->h_words != nullptr) cudaFreeHost(g->h_words);
    if (g->stream != nullptr) cudaStreamDestroy(g->stream);
    delete g;
}

}  // namespace

extern "C" {

// ---- model ---------------------------------------------------------------------------------------

mc_status_t mc_sm100_model_load(const char* model_dir, const mc_sm100_model_options_t* o, mc_sm100_model_t* out_model) {
    MC_TRY
    clear_error();
    if (out_model != nullptr) *out_model = mc_sm100_model_t{nullptr};
    if (model_dir == nullptr) { set_error("mc_sm100_model_load: model_dir is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (o == nullptr) { set_error("mc_sm100_model_load: options is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (out_model == nullptr) { set_error("mc_sm100_model_load: out_model is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (o->struct_size != sizeof(*o)) {
        set_error("mc_sm100_model_load: options->struct_size=%u but expected %zu", o->struct_size, sizeof(*o));
        return MC_E_INVALID_ARGUMENT;
    }
    if (o->abi_version != MC_SM100_ABI_VERSION) {
        set_error("mc_sm100_model_load: options->abi_version=0x%08x but expected 0x%08x", o->abi_version, MC_SM100_ABI_VERSION);
        return MC_E_INVALID_ARGUMENT;
    }
    if (o->reserved0 != 0 || o->reserved[0] != 0 || o->reserved[1] != 0 || o->reserved[2] != 0 || o->reserved[3] != 0) {
        set_error("mc_sm100_model_load: reserved fields must be zero");
        return MC_E_INVALID_ARGUMENT;
    }
    if (o->precision != 0u && o->precision != 2u) {
        set_error("mc_sm100_model_load: only bf16 (0) and e4m3 weight-only (2) are supported (options->precision=%u)", o->precision);
        return MC_E_UNSUPPORTED;
    }
    if (o->max_sessions == 0 || o->max_sessions > kMaxSlots) {
        set_error("mc_sm100_model_load: max_sessions=%u out of range [1,%u]", o->max_sessions, kMaxSlots);
        return MC_E_INVALID_ARGUMENT;
    }
    if (!dir_exists(model_dir)) { set_error("mc_sm100_model_load: model directory '%s' does not exist", model_dir); return MC_E_IO; }
    mc_status_t rc = MC_OK;
    mc_sm100_model_impl* m = new (std::nothrow) mc_sm100_model_impl();
    if (m == nullptr) { set_error("mc_sm100_model_load: out of host memory"); return MC_E_OUT_OF_MEMORY; }
    m->device = o->device_id; m->precision = o->precision; m->graph = o->enable_cuda_graph; m->max_sessions = o->max_sessions;
    m->d_weights = nullptr; m->d_embedding = nullptr; m->sessions.store(0);

    const std::string wpk_path = std::string(model_dir) + "/model.wpk";
    mc_sm100_wpk_t wpk = nullptr;
    if (file_exists(wpk_path)) {
        rc = mc_sm100_wpk_open(wpk_path.c_str(), &wpk);
        if (rc != MC_OK) { delete m; return rc; }
        mc_sm100_wpk_section_t emb{}, qkv{}, gu{};
        rc = mc_sm100_wpk_find(wpk, "embedding", &emb);
        if (rc == MC_OK) rc = mc_sm100_wpk_find(wpk, "layer0.qkv", &qkv);
        if (rc == MC_OK) rc = mc_sm100_wpk_find(wpk, "layer0.gate_up", &gu);
        if (rc == MC_OK && (emb.rank != 2 || qkv.rank != 2 || gu.rank != 2 || qkv.dims[1] != emb.dims[1] || gu.dims[1] != emb.dims[1] ||
                            (gu.dims[0] & 1u) != 0 || emb.dtype != 0)) {
            set_error("mc_sm100_model_load: inconsistent section shapes in %s", wpk_path.c_str());
            rc = MC_E_MODEL_MISMATCH;
        }
        if (rc == MC_OK && qkv.dtype != o->precision) {
            set_error("mc_sm100_model_load: %s holds dtype %u matrices but options->precision is %u", wpk_path.c_str(), qkv.dtype, o->precision);
            rc = MC_E_MODEL_MISMATCH;
        }
        if (rc != MC_OK) { mc_sm100_wpk_close(wpk); delete m; return rc; }
        m->V = emb.dims[0]; m->H = emb.dims[1]; m->Q = qkv.dims[0]; m->I = gu.dims[0] / 2u;
        uint32_t layers = 0;
        for (;; ++layers) {
            char name[64];
            std::snprintf(name, sizeof(name), "layer%u.qkv", layers);
            mc_sm100_wpk_section_t t{};
            if (mc_sm100_wpk_find(wpk, name, &t) != MC_OK) break;
        }
        clear_error();
        m->L = layers;
    } else {
        m->L = o->synth_layers; m->H = o->synth_hidden; m->Q = o->synth_qkv_rows; m->I = o->synth_inter; m->V = o->synth_vocab;
    }
    const mc_sm100_stack_desc_t d = m->desc(1);
    uint64_t wbytes = 0, sbytes = 0;
    rc = mc_sm100_stack_sizes(&d, &wbytes, &sbytes);
    if (rc != MC_OK) {
        set_error("mc_sm100_model_load: unsupported model dimensions (layers=%u hidden=%u qkv=%u inter=%u vocab=%u)", m->L, m->H, m->Q, m->I, m->V);
        if (wpk != nullptr) mc_sm100_wpk_close(wpk);
        delete m;
        return wpk != nullptr ? MC_E_MODEL_MISMATCH : MC_E_INVALID_ARGUMENT;
    }
    m->weight_bytes = wbytes;
    // everything above was host-side validation; from here on the device is needed
    cudaError_t e = cudaSetDevice(o->device_id);
    if (e == cudaSuccess) {
        rc = mc_sm100_device_check(nullptr, nullptr, nullptr, nullptr);    // compute capability 10.x (model.cpp:133-139 wants 12.0)
        if (rc != MC_OK) { if (wpk != nullptr) mc_sm100_wpk_close(wpk); delete m; return rc; }
        e = cudaMalloc(reinterpret_cast<void**>(&m->d_weights), wbytes);
    }
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&m->d_embedding), (size_t)m->V * m->H * 2u);
    if (e == cudaSuccess) e = cudaMemset(m->d_weights, 0, wbytes);
    if (e != cudaSuccess) {
        if (wpk != nullptr) mc_sm100_wpk_close(wpk);
        rc = cuda_fail("mc_sm100_model_load", "weight arena allocation", e);
        release_model(m);
        return rc;
    }
    m->vram_bytes = wbytes + (uint64_t)m->V * m->H * 2u;
    rc = wpk != nullptr ? upload_wpk(m, wpk) : fill_synthetic(m, o->synth_seed);
    if (wpk != nullptr) mc_sm100_wpk_close(wpk);
    if (rc != MC_OK) { release_model(m); return rc; }
    *out_model = mc_sm100_model_t{m};
    return MC_OK;
    MC_CATCH("mc_sm100_model_load")
}

void mc_sm100_model_destroy(mc_sm100_model_t model) {
    if (model.impl == nullptr) return;
    (void)cudaSetDevice(model.impl->device);
    release_model(model.impl);
}

mc_status_t mc_sm100_debug_model_dims(mc_sm100_model_t model, uint32_t* layers, uint32_t* hidden, uint32_t* qkv_rows, uint32_t* inter,
                                      uint32_t* vocab) {
    clear_error();
    if (model.impl == nullptr) { set_error("mc_sm100_debug_model_dims: model is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (layers) *layers = model.impl->L;
    if (hidden) *hidden = model.impl->H;
    if (qkv_rows) *qkv_rows = model.impl->Q;
    if (inter) *inter = model.impl->I;
    if (vocab) *vocab = model.impl->V;
    return MC_OK;
}

// ---- session -------------------------------------------------------------------------------------

mc_status_t mc_sm100_session_create(mc_sm100_model_t model, mc_sm100_session_t* out_session) {
    MC_TRY
    clear_error();
    if (out_session != nullptr) *out_session = mc_sm100_session_t{nullptr};
    if (model.impl == nullptr) { set_error("mc_sm100_session_create: model is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (out_session == nullptr) { set_error("mc_sm100_session_create: out_session is NULL"); return MC_E_INVALID_ARGUMENT; }
    mc_sm100_model_impl* m = model.impl;
    if (m->sessions.fetch_add(1) >= m->max_sessions) {
        m->sessions.fetch_sub(1);
        set_error("mc_sm100_session_create: the model serves at most %u sessions", m->max_sessions);
        return MC_E_UNSUPPORTED;
    }
    cudaError_t e = cudaSetDevice(m->device);
    mc_sm100_session_impl* s = new (std::nothrow) mc_sm100_session_impl();
    if (s == nullptr) { m->sessions.fetch_sub(1); set_error("mc_sm100_session_create: out of host memory"); return MC_E_OUT_OF_MEMORY; }
    std::memset(static_cast<void*>(s), 0, sizeof(*s));
    s->model = m;
    const mc_sm100_stack_desc_t d = m->desc(1);
    uint64_t wbytes = 0, sbytes = 0;
    mc_status_t rc = mc_sm100_stack_sizes(&d, &wbytes, &sbytes);
    if (rc != MC_OK) { release_session(s); return rc; }
    const size_t x_off = align256(sbytes), tok_off = x_off + align256((size_t)m->H * 2u), total = tok_off + 256u;
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&s->d_block), total);
    if (e == cudaSuccess) e = cudaMemset(s->d_block, 0, total);
    if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&s->h_word), 64, cudaHostAllocDefault);
    if (e != cudaSuccess) { rc = cuda_fail("mc_sm100_session_create", "allocation", e); release_session(s); return rc; }
    s->d_x = reinterpret_cast<uint16_t*>(s->d_block + x_off);
    s->d_next_token = reinterpret_cast<int32_t*>(s->d_block + tok_off);
    s->d_emitted = s->d_next_token + 1;
    rc = mc_sm100_stack_create(&d, m->d_weights, s->d_block, &s->stack);
    if (rc != MC_OK) { release_session(s); return rc; }
    *out_session = mc_sm100_session_t{s};
    return MC_OK;
    MC_CATCH("mc_sm100_session_create")
}

mc_status_t mc_sm100_session_reset(mc_sm100_session_t session) {
    MC_TRY
    clear_error();
    mc_sm100_session_impl* s = session.impl;
    if (s == nullptr) { set_error("mc_sm100_session_reset: session is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (s->group != nullptr) { set_error("mc_sm100_session_reset: session is a member of a batch group"); return MC_E_UNSUPPORTED; }
    (void)cudaSetDevice(s->model->device);
    const cudaError_t e = cudaStreamSynchronize(s->stream);
    if (e != cudaSuccess) return cuda_fail("mc_sm100_session_reset", "stream synchronise", e);
    s->seq_len = 0;
    std::memset(&s->stats, 0, sizeof(s->stats));
    return MC_OK;
    MC_CATCH("mc_sm100_session_reset")
}

void mc_sm100_session_destroy(mc_sm100_session_t session) {
    if (session.impl == nullptr) return;
    (void)cudaSetDevice(session.impl->model->device);
    release_session(session.impl);
}

// one solo step on the session's stream: eager the first time, then the captured graph
static mc_status_t session_step(mc_sm100_session_impl* s, const char* who) {
    const mc_sm100_model_impl* m = s->model;
    auto body = [&]() { return enqueue_step(m, s->stack, nullptr, s->d_next_token, s->d_x, s->d_emitted, s->d_next_token, 1u, s->stream); };
    if (m->graph && s->graph != nullptr) {
        const cudaError_t e = cudaGraphLaunch(s->graph, s->stream);
        if (e != cudaSuccess) { (void)cudaGetLastError(); set_error("%s: graph launch failed: %s", who, cudaGetErrorString(e)); return MC_E_GRAPH; }
        s->stats.cuda_graph_launches += 1;
        return MC_OK;
    }
    const mc_status_t rc = body();
    if (rc != MC_OK) return rc;
    if (m->graph && s->graph == nullptr) capture_graph(s->stream, &s->graph, body);   // for the steps that follow
    return MC_OK;
}

// emitted token + failure word to the host, one synchronise
static mc_status_t session_harvest(mc_sm100_session_impl* s, const char* who, int32_t* out_token) {
    cudaError_t e = cudaMemcpyAsync(&s->h_word[0], s->d_emitted, 4, cudaMemcpyDeviceToHost, s->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&s->h_word[1], mc_sm100_stack_status_word(s->stack), 4, cudaMemcpyDeviceToHost, s->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
    if (e != cudaSuccess) return cuda_fail(who, "token D2H / stream synchronise", e);
    if (s->h_word[1] != 0) { set_error("%s: a bounded wait ran out inside a kernel of the step", who); return MC_E_INTERNAL; }
    if (out_token != nullptr) {
        const int32_t tok = s->h_word[0];
        if (tok < 0 || (uint32_t)tok >= s->model->V) { set_error("%s: the step emitted the out-of-range token %d", who, tok); return MC_E_INTERNAL; }
        *out_token = tok;
    }
    return MC_OK;
}

mc_status_t mc_sm100_prefill(mc_sm100_session_t session, const int32_t* token_ids, uint32_t token_count) {
    MC_TRY
    clear_error();
    mc_sm100_session_impl* s = session.impl;
    if (s == nullptr) { set_error("mc_sm100_prefill: session is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (token_ids == nullptr || token_count == 0) { set_error("mc_sm100_prefill: token_ids is NULL or token_count is 0"); return MC_E_INVALID_ARGUMENT; }
    if (s->group != nullptr) { set_error("mc_sm100_prefill: session is a member of a batch group"); return MC_E_UNSUPPORTED; }
    for (uint32_t i = 0; i < token_count; ++i)
        if (token_ids[i] < 0 || (uint32_t)token_ids[i] >= s->model->V) {
            set_error("mc_sm100_prefill: token_ids[%u]=%d outside [0,%u)", i, token_ids[i], s->model->V);
            return MC_E_INVALID_ARGUMENT;
        }
    (void)cudaSetDevice(s->model->device);
    const auto t0 = std::chrono::steady_clock::now();
    s->h_word[2] = token_ids[token_count - 1];
    const cudaError_t e = cudaMemcpyAsync(s->d_next_token, &s->h_word[2], 4, cudaMemcpyHostToDevice, s->stream);
    if (e != cudaSuccess) return cuda_fail("mc_sm100_prefill", "token H2D", e);
    mc_status_t rc = session_step(s, "mc_sm100_prefill");
    if (rc == MC_OK) rc = session_harvest(s, "mc_sm100_prefill", nullptr);
    if (rc != MC_OK) return rc;
    s->seq_len = token_count;
    s->stats.prompt_tokens += token_count;
    s->stats.prefill_us += (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
    return MC_OK;
    MC_CATCH("mc_sm100_prefill")
}

mc_status_t mc_sm100_decode_one(mc_sm100_session_t session, const mc_sm100_generation_config_t* config, int32_t* out_token) {
    MC_TRY
    clear_error();
    mc_sm100_session_impl* s = session.impl;
    if (s == nullptr) { set_error("mc_sm100_decode_one: session is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (config == nullptr || out_token == nullptr) { set_error("mc_sm100_decode_one: config/out_token is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (config->struct_size != sizeof(*config)) {
        set_error("mc_sm100_decode_one: config->struct_size=%u but expected %zu", config->struct_size, sizeof(*config));
        return MC_E_INVALID_ARGUMENT;
    }
    if (s->seq_len == 0) { set_error("mc_sm100_decode_one: sequence is empty (prefill first)"); return MC_E_INVALID_ARGUMENT; }
    if (s->group != nullptr) { set_error("mc_sm100_decode_one: session is a member of a batch group"); return MC_E_UNSUPPORTED; }
    if (!greedy_only(*config)) { set_error("mc_sm100_decode_one: only greedy decoding on this entry point"); return MC_E_UNSUPPORTED; }
    (void)cudaSetDevice(s->model->device);
    const auto t0 = std::chrono::steady_clock::now();
    mc_status_t rc = session_step(s, "mc_sm100_decode_one");
    if (rc == MC_OK) rc = session_harvest(s, "mc_sm100_decode_one", out_token);
    if (rc != MC_OK) return rc;
    s->seq_len += 1;
    s->stats.generated_tokens += 1;
    s->stats.decode_us += (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
    return MC_OK;
    MC_CATCH("mc_sm100_decode_one")
}

mc_status_t mc_sm100_get_stats(mc_sm100_session_t session, mc_sm100_runtime_stats_t* out_stats) {
    clear_error();
    if (session.impl == nullptr || out_stats == nullptr) { set_error("mc_sm100_get_stats: session/out_stats is NULL"); return MC_E_INVALID_ARGUMENT; }
    *out_stats = session.impl->stats;
    out_stats->peak_vram_bytes = session.impl->model->vram_bytes;
    return MC_OK;
}

mc_status_t mc_sm100_debug_session_logits(mc_sm100_session_t session, uint16_t* h_logits, uint32_t count) {
    MC_TRY
    clear_error();
    mc_sm100_session_impl* s = session.impl;
    if (s == nullptr || h_logits == nullptr || count == 0 || count > s->model->V) { set_error("mc_sm100_debug_session_logits: invalid args"); return MC_E_INVALID_ARGUMENT; }
    (void)cudaSetDevice(s->model->device);
    cudaError_t e = cudaMemcpyAsync(h_logits, mc_sm100_stack_logits(s->stack), (size_t)count * 2u, cudaMemcpyDeviceToHost, s->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
    if (e != cudaSuccess) return cuda_fail("mc_sm100_debug_session_logits", "logits D2H", e);
    return MC_OK;
    MC_CATCH("mc_sm100_debug_session_logits")
}

// ---- batch group -----------------------------------------------------------------------------------

mc_status_t mc_sm100_batch_group_create(mc_sm100_model_t model, const mc_sm100_batch_options_t* o, mc_sm100_batch_group_t* out_group) {
    MC_TRY
    clear_error();
    if (out_group != nullptr) *out_group = mc_sm100_batch_group_t{nullptr};
    if (model.impl == nullptr) { set_error("mc_sm100_batch_group_create: model is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (o == nullptr || out_group == nullptr) { set_error("mc_sm100_batch_group_create: options/out_group is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (o->struct_size != sizeof(*o)) {
        set_error("mc_sm100_batch_group_create: options->struct_size=%u but expected %zu", o->struct_size, sizeof(*o));
        return MC_E_INVALID_ARGUMENT;
    }
    if (o->abi_version != MC_SM100_ABI_VERSION) {
        set_error("mc_sm100_batch_group_create: abi_version=0x%08x expected 0x%08x", o->abi_version, MC_SM100_ABI_VERSION);
        return MC_E_INVALID_ARGUMENT;
    }
    for (uint32_t i = 0; i < 4; ++i)
        if (o->reserved[i] != 0) { set_error("mc_sm100_batch_group_create: reserved[%u] must be zero", i); return MC_E_INVALID_ARGUMENT; }
    if (o->max_slots == 0 || o->max_slots > kMaxSlots) {
        set_error("mc_sm100_batch_group_create: max_slots=%u out of range [1,%u]", o->max_slots, kMaxSlots);
        return MC_E_UNSUPPORTED;
    }
    mc_sm100_model_impl* m = model.impl;
    cudaError_t e = cudaSetDevice(m->device);
    if (e != cudaSuccess) return cuda_fail("mc_sm100_batch_group_create", "cudaSetDevice", e);
    mc_sm100_batch_group_impl* g = new (std::nothrow) mc_sm100_batch_group_impl();
    if (g == nullptr) { set_error("mc_sm100_batch_group_create: out of host memory"); return MC_E_OUT_OF_MEMORY; }
    std::memset(static_cast<void*>(g), 0, sizeof(*g));
    g->model = m;
    g->max_slots = o->max_slots;
    const mc_sm100_stack_desc_t d = m->desc(g->max_slots);
    uint64_t wbytes = 0, sbytes = 0;
    mc_status_t rc = mc_sm100_stack_sizes(&d, &wbytes, &sbytes);
    if (rc != MC_OK) { release_group(g); return rc; }
    const size_t R = g->max_slots;
    const size_t x_off = align256(sbytes), tok_off = x_off + align256(R * m->H * 2u), emit_off = tok_off + align256(R * 4u),
                 tab_off = emit_off + align256(R * 4u), total = tab_off + align256(R * 8u);
    e = cudaStreamCreateWithFlags(&g->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&g->d_block), total);
    if (e == cudaSuccess) e = cudaMemset(g->d_block, 0, total);
    if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&g->h_step_tok), kMaxSlots * sizeof(void*), cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&g->h_words), (kMaxSlots + 1) * 4u, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&g->ev_group, cudaEventDisableTiming);
    for (uint32_t i = 0; i < g->max_slots && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&g->ev_member[i], cudaEventDisableTiming);
    if (e != cudaSuccess) { rc = cuda_fail("mc_sm100_batch_group_create", "allocation", e); release_group(g); return rc; }
    g->d_x = reinterpret_cast<uint16_t*>(g->d_block + x_off);
    g->d_tokens = reinterpret_cast<int32_t*>(g->d_block + tok_off);
    g->d_emitted = reinterpret_cast<int32_t*>(g->d_block + emit_off);
    g->d_step_tok = reinterpret_cast<int32_t**>(g->d_block + tab_off);
    rc = mc_sm100_stack_create(&d, m->d_weights, g->d_block, &g->stack);
    if (rc != MC_OK) { release_group(g); return rc; }
    *out_group = mc_sm100_batch_group_t{g};
    return MC_OK;
    MC_CATCH("mc_sm100_batch_group_create")
}

mc_status_t mc_sm100_batch_group_add(mc_sm100_batch_group_t group, mc_sm100_session_t session, uint32_t* slot_id) {
    MC_TRY
    clear_error();
    mc_sm100_batch_group_impl* g = group.impl;
    if (g == nullptr) { set_error("mc_sm100_batch_group_add: group is NULL"); return MC_E_INVALID_ARGUMENT; }
    mc_sm100_session_impl* s = session.impl;
    if (s == nullptr || slot_id == nullptr) { set_error("mc_sm100_batch_group_add: session/slot_id is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (s->model != g->model) { set_error("mc_sm100_batch_group_add: session belongs to a different model"); return MC_E_UNSUPPORTED; }
    if (s->group != nullptr) { set_error("mc_sm100_batch_group_add: session is already in a batch group"); return MC_E_UNSUPPORTED; }
    uint32_t slot = g->max_slots;
    for (uint32_t i = 0; i < g->max_slots; ++i)
        if (g->members[i] == nullptr) { slot = i; break; }
    if (slot == g->max_slots) { set_error("mc_sm100_batch_group_add: group is full (max_slots=%u)", g->max_slots); return MC_E_UNSUPPORTED; }
    (void)cudaSetDevice(g->model->device);
    // member stream -> group stream: the member's earlier prefill / solo steps are visible to the group
    cudaError_t e = cudaEventRecord(g->ev_member[slot], s->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(g->stream, g->ev_member[slot], 0);
    if (e != cudaSuccess) return cuda_fail("mc_sm100_batch_group_add", "event chain (member->group)", e);
    g->members[slot] = s;
    s->group = g;
    *slot_id = slot;
    return MC_OK;
    MC_CATCH("mc_sm100_batch_group_add")
}

static mc_status_t group_remove(mc_sm100_batch_group_impl* g, uint32_t slot_id, const char* who) {
    mc_sm100_session_impl* s = g->members[slot_id];
    // group stream -> member stream: the group's token writes are visible to the member's next solo call
    cudaError_t e = cudaEventRecord(g->ev_group, g->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s->stream, g->ev_group, 0);
    if (e != cudaSuccess) return cuda_fail(who, "event chain (group->member)", e);
    g->members[slot_id] = nullptr;
    s->group = nullptr;
    return MC_OK;
}

mc_status_t mc_sm100_batch_group_remove(mc_sm100_batch_group_t group, uint32_t slot_id) {
    MC_TRY
    clear_error();
    mc_sm100_batch_group_impl* g = group.impl;
    if (g == nullptr) { set_error("mc_sm100_batch_group_remove: group is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (slot_id >= g->max_slots || g->members[slot_id] == nullptr) {
        set_error("mc_sm100_batch_group_remove: slot %u has no member", slot_id);
        return MC_E_INVALID_ARGUMENT;
    }
    (void)cudaSetDevice(g->model->device);
    return group_remove(g, slot_id, "mc_sm100_batch_group_remove");
    MC_CATCH("mc_sm100_batch_group_remove")
}

mc_status_t mc_sm100_batch_step(mc_sm100_batch_group_t group, const uint32_t* slot_ids, uint32_t n,
                                const mc_sm100_generation_config_t* cfgs, int32_t* out_tokens) {
    MC_TRY
    clear_error();
    mc_sm100_batch_group_impl* g = group.impl;
    if (g == nullptr) { set_error("mc_sm100_batch_step: group is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (slot_ids == nullptr || cfgs == nullptr || out_tokens == nullptr) { set_error("mc_sm100_batch_step: slot_ids/cfgs/out_tokens is NULL"); return MC_E_INVALID_ARGUMENT; }
    if (n == 0 || n > g->max_slots) { set_error("mc_sm100_batch_step: n=%u out of range [1,%u]", n, g->max_slots); return MC_E_INVALID_ARGUMENT; }
    for (uint32_t i = 0; i < n; ++i) {
        const uint32_t sid = slot_ids[i];
        if (sid >= g->max_slots || g->members[sid] == nullptr) { set_error("mc_sm100_batch_step: slot_ids[%u]=%u has no member", i, sid); return MC_E_INVALID_ARGUMENT; }
        for (uint32_t j = 0; j < i; ++j)
            if (slot_ids[j] == sid) { set_error("mc_sm100_batch_step: duplicate slot %u", sid); return MC_E_INVALID_ARGUMENT; }
        if (cfgs[i].struct_size != sizeof(cfgs[i])) {
            set_error("mc_sm100_batch_step: cfgs[%u].struct_size=%u but expected %zu", i, cfgs[i].struct_size, sizeof(cfgs[i]));
            return MC_E_INVALID_ARGUMENT;
        }
        if (!greedy_only(cfgs[i])) { set_error("mc_sm100_batch_step: non-greedy cfgs[%u] unsupported on this entry point", i); return MC_E_UNSUPPORTED; }
        if (g->members[sid]->seq_len == 0) { set_error("mc_sm100_batch_step: slot %u sequence is empty (prefill first)", sid); return MC_E_INVALID_ARGUMENT; }
    }
    const mc_sm100_model_impl* m = g->model;
    (void)cudaSetDevice(m->device);
    const cudaStream_t st = g->stream;
    const auto t0 = std::chrono::steady_clock::now();
    // step table: where each row's token lives (fixed table address, contents refreshed by a small H2D)
    for (uint32_t i = 0; i < n; ++i) g->h_step_tok[i] = g->members[slot_ids[i]]->d_next_token;
    cudaError_t e = cudaMemcpyAsync(g->d_step_tok, g->h_step_tok, (size_t)n * sizeof(void*), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return cuda_fail("mc_sm100_batch_step", "step table H2D", e);
    auto body = [&]() {
        return enqueue_step(m, g->stack, (const int32_t* const*)g->d_step_tok, nullptr, g->d_x, g->d_emitted, g->d_tokens, n, st);
    };
    if (m->graph && g->graph[n] != nullptr) {
        e = cudaGraphLaunch(g->graph[n], st);
        if (e != cudaSuccess) { (void)cudaGetLastError(); set_error("mc_sm100_batch_step: graph launch failed: %s", cudaGetErrorString(e)); return MC_E_GRAPH; }
    } else {
        const mc_status_t rc = body();
        if (rc != MC_OK) return rc;
        if (m->graph) {
            capture_graph(st, &g->graph[n], body);      // one graph per batch size, for the steps that follow
            if (g->graph[n] != nullptr) g->graphs += 1;
        }
    }
    e = cudaMemcpyAsync(g->h_words, g->d_emitted, (size_t)n * 4u, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&g->h_words[kMaxSlots], mc_sm100_stack_status_word(g->stack), 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail("mc_sm100_batch_step", "token D2H / stream synchronise", e);
    if (g->h_words[kMaxSlots] != 0) { set_error("mc_sm100_batch_step: a bounded wait ran out inside a kernel of the step"); return MC_E_INTERNAL; }
    for (uint32_t i = 0; i < n; ++i) {
        const int32_t tok = g->h_words[i];
        if (tok < 0 || (uint32_t)tok >= m->V) { set_error("mc_sm100_batch_step: slot %u emitted out-of-range token %d", slot_ids[i], tok); return MC_E_INTERNAL; }
        out_tokens[i] = tok;
    }
    for (uint32_t i = 0; i < n; ++i) {
        mc_sm100_session_impl* s = g->members[slot_ids[i]];
        s->seq_len += 1;
        s->stats.generated_tokens += 1;
    }
    g->decode_us += (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
    g->steps += 1;
    return MC_OK;
    MC_CATCH("mc_sm100_batch_step")
}

void mc_sm100_batch_group_destroy(mc_sm100_batch_group_t group) {
    mc_sm100_batch_group_impl* g = group.impl;
    if (g == nullptr) return;
    (void)cudaSetDevice(g->model->device);
    for (uint32_t i = 0; i < g->max_slots; ++i)
        if (g->members[i] != nullptr) (void)group_remove(g, i, "mc_sm100_batch_group_destroy");
    release_group(g);
}

mc_status_t mc_sm100_debug_batch_group_stats(mc_sm100_batch_group_t group, uint64_t* steps, uint64_t* decode_us, uint32_t* members,
                                             uint32_t* graphs) {
    clear_error();
    mc_sm100_batch_group_impl* g = group.impl;
    if (g == nullptr) { set_error("mc_sm100_debug_batch_group_stats: group is NULL"); return MC_E_INVALID_ARGUMENT; }
    uint32_t live = 0;
    for (uint32_t i = 0; i < g->max_slots; ++i) live += g->members[i] != nullptr ? 1u : 0u;
    if (steps) *steps = g->steps;
    if (decode_us) *decode_us = g->decode_us;
    if (members) *members = live;
    if (graphs) *graphs = g->graphs;
    return MC_OK;
}

}  // extern "C"
