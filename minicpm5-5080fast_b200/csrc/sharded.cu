// sharded.cu -- M = 1 linears whose output exchange between GPUs runs inside the GEMV.
//
// A column-parallel (N-sharded) decode step needs the whole output vector of every linear
// on every rank before the next linear can start.  At M = 1 those vectors are 0.6 - 11 KB,
// so a separate collective per linear (a library all-gather, or even one small peer-copy
// kernel) costs more than the sharded GEMV it follows, and so does any flag protocol that
// needs a system-scope fence (measured on two B200s: ~3 us per fence, ~9 us per exchange
// with a fence and a remote atomic per CTA, 3.3 us with one flag store by the last CTA).
// Here the producing GEMV stores every output element directly into all ranks' gathered
// vectors over NVLink as a self-validating 32-bit word (value + sequence tag, one
// destination rank per lane) and the consuming GEMV -- whose weights are already in flight
// -- polls the words while it stages the activation.  Nothing else runs between two
// linears.  All waits are bounded in time and sticky on failure.
#include "fast_dispatch.cuh"

namespace mcl {

// One CTA.  Every rank pushes the (value, index) of each of its n_rows shard results to every rank
// (pair slots laid out [world][n_rows]), signals, waits -- bounded -- for the others, then reduces
// each row over the ranks with the reference's tie rule and advances *step.
__global__ void __launch_bounds__(256, 1)
peer_argmax_kernel(const float* __restrict__ val, const int32_t* __restrict__ idx, uint32_t n_rows,
                   const uint64_t* __restrict__ pair_peers, const uint64_t* __restrict__ flag_peers, const uint64_t* my_pairs,
                   const uint32_t* my_flags, uint32_t* step, uint32_t rank, uint32_t world, unsigned long long limit_ns,
                   int32_t* status, int32_t* token, float* token_val) {
    __shared__ uint32_t s_step;
    __shared__ int s_ok;
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x == 0) { s_step = *step; s_ok = 1; }
    __syncthreads();
    const uint32_t s = s_step;
    for (uint32_t i = threadIdx.x; i < world * n_rows; i += blockDim.x) {
        const uint32_t p = i / n_rows, m = i - p * n_rows;
        const uint64_t packed = (uint64_t)__float_as_uint(val[m]) | ((uint64_t)(uint32_t)idx[m] << 32);
        *reinterpret_cast<volatile uint64_t*>(reinterpret_cast<uint64_t*>(pair_peers[p]) + (size_t)rank * n_rows + m) = packed;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
        const uint64_t f = flag_peers[threadIdx.x] + 4ull * rank;
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(f), "r"(1u) : "memory");
        const uint32_t* mine = my_flags + threadIdx.x;
        unsigned long long t0 = 0;
        bool ok = *reinterpret_cast<volatile int32_t*>(status) == 0;
        for (uint32_t spin = 0; ok; ++spin) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - s) >= 0) break;
            if ((spin & 31u) == 31u) {
                const unsigned long long now = global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > limit_ns) { *reinterpret_cast<volatile int32_t*>(status) = 1; ok = false; }
            }
        }
        if (!ok) s_ok = 0;
    }
    __syncthreads();
    for (uint32_t m = threadIdx.x; m < n_rows; m += blockDim.x) {
        float bv = -INFINITY;
        int32_t bi = INT32_MAX;
        if (s_ok) {
            for (uint32_t r = 0; r < world; ++r) {
                const uint64_t got = *reinterpret_cast<const volatile uint64_t*>(my_pairs + (size_t)r * n_rows + m);
                const float v = __uint_as_float((uint32_t)got);
                const int32_t i = (int32_t)(uint32_t)(got >> 32);
                if (v == v && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
            }
        }
        token[m] = bi;
        if (token_val != nullptr) token_val[m] = bv;
    }
    if (threadIdx.x == 0) *step = s + 1u;
}

}  // namespace mcl

using namespace mcl;

extern "C" {

mc_status_t mc_sm100_gemv_sharded(int32_t prologue, int32_t epilogue, const void* d_w, const float* d_scale,
                                  const uint16_t* d_x, const uint16_t* d_addend, const uint16_t* d_norm_w,
                                  uint16_t* d_res_out, uint16_t* d_y, uint32_t N, uint32_t K, float eps,
                                  const mc_sm100_shard_io_t* io, void* stream, int32_t pdl) {
    clear_error();
    const int wb = d_scale == nullptr ? 2 : 1;
    if (io == nullptr || d_w == nullptr || d_x == nullptr || N == 0 || K == 0 || (K % (wb == 2 ? 8u : 16u)) != 0 ||
        !aligned16(d_w) || !aligned16(d_x) || (prologue != 0 && prologue != 1) || (epilogue != 0 && epilogue != 1) ||
        (epilogue == 1 && (N & 1u) != 0) || (io->out_slot == 0 && d_y == nullptr) || (io->in_tagged && prologue == 1 && d_addend == nullptr) ||
        (prologue == 1 && (d_norm_w == nullptr || d_res_out == nullptr || d_res_out == d_x))) {
        set_error("mc_sm100_gemv_sharded: invalid args (N=%u K=%u prologue=%d epilogue=%d)", N, K, prologue, epilogue);
        return MC_E_INVALID_ARGUMENT;
    }
    const uint32_t outs = epilogue == 1 ? N / 2u : N;
    RowsArgs a{};
    const mc_status_t rc = shard_io_to_args("mc_sm100_gemv_sharded", io, outs, true, a.sh);
    if (rc != MC_OK) return rc;
    a.w = d_w; a.scale = d_scale; a.y = d_y; a.N = N; a.K = K; a.y_stride = outs; a.kseg = K;
    if (prologue == 1) { a.res_in = d_x; a.addend = d_addend; a.norm_w = d_norm_w; a.res_out = d_res_out; a.eps = eps; }
    else a.x = d_x;
    const NextWeights nw = take_next_weights();
    a.pf.ptr = static_cast<const uint8_t*>(nw.ptr); a.pf.bytes = nw.bytes;
    const int pro = prologue == 1 ? PRO_RESNORM : PRO_NONE, epi = epilogue == 1 ? EPI_SWIGLU : EPI_STORE;
    return wb == 2 ? launch_fast<2>(pro, epi, a, (cudaStream_t)stream, pdl != 0)
                   : launch_fast<1>(pro, epi, a, (cudaStream_t)stream, pdl != 0);
}

mc_status_t mc_sm100_peer_argmax(const float* d_val, const int32_t* d_idx, uint32_t n_rows, const uint64_t* d_pair_peers,
                                 const uint64_t* d_flag_peers, const uint64_t* d_my_pairs, const uint32_t* d_my_flags,
                                 uint32_t* d_step, uint32_t rank, uint32_t world, uint64_t timeout_ns,
                                 int32_t* d_status, int32_t* d_token, float* d_token_val, void* stream, int32_t pdl) {
    clear_error();
    if (d_val == nullptr || d_idx == nullptr || d_pair_peers == nullptr || d_flag_peers == nullptr ||
        d_my_pairs == nullptr || d_my_flags == nullptr || d_step == nullptr || d_status == nullptr ||
        d_token == nullptr || world == 0 || world > 32u || rank >= world || n_rows == 0 || n_rows > 64u) {
        set_error("mc_sm100_peer_argmax: invalid args (rank=%u world=%u rows=%u)", rank, world, n_rows);
        return MC_E_INVALID_ARGUMENT;
    }
    (void)launch(peer_argmax_kernel, dim3(1), dim3(256), 0, (cudaStream_t)stream, pdl != 0, d_val, d_idx, n_rows, d_pair_peers,
                 d_flag_peers, d_my_pairs, d_my_flags, d_step, rank, world,
                 (unsigned long long)(timeout_ns ? timeout_ns : kShardWaitDefaultNs), d_status, d_token, d_token_val);
    MCL_CHECK_LAUNCH("peer_argmax");
    return MC_OK;
}

}  // extern "C"
