// peer_gather.cu -- all-gather of an N-shard over NVLink peer memory, one small kernel.
//
// After a sharded linear every rank holds its slice of the output and every rank needs
// the whole vector for the next linear.  The slices are tiny (0.6 - 30 KB), so a
// library collective costs several times the sharded GEMV itself.  Here each rank's
// kernel stores its slice straight into every rank's gathered buffer through peer-mapped
// pointers (plain 16-byte stores, no TMA, no multicast), publishes an epoch number in
// every rank's flag array with a system-scope release, and then waits -- bounded in
// time -- until all ranks' flags have reached the same epoch.  The epoch lives in device
// memory and is advanced by the kernel itself, so a captured graph can be replayed.
// A rank can be at most one exchange ahead of its slowest peer (its next exchange needs
// that peer's flag), so buffers that rotate with a period of two or more are never
// overwritten while a peer still reads them.
#include "common.cuh"

namespace mcl {

constexpr unsigned long long kPeerWaitDefaultNs = 1000ull * 1000ull * 1000ull;   // 1 s

// rows x row_units (16-byte units) from a contiguous shard to column slot `rank` of every peer's
// buffer, whose rows are pitch_units apart (rows = 1: the plain 1-D gather).
__global__ void __launch_bounds__(512, 1)
peer_allgather_kernel(const uint4* __restrict__ shard, uint32_t rows, uint32_t row_units, uint32_t pitch_units, uint32_t slot_units,
                      const uint64_t* __restrict__ peer_bufs, const uint64_t* __restrict__ peer_flags,
                      uint32_t* my_flags, uint32_t* epoch, uint32_t rank, uint32_t world,
                      unsigned long long limit_ns, int32_t* status) {
    __shared__ uint32_t s_epoch;
    __shared__ int s_fail, s_dead;
    pdl_trigger();
    pdl_wait();
    // sticky failure: once a wait has run out (a peer fell behind or left) no later gather waits
    // again -- it still pushes its slice and advances the epoch, so a replayed graph stays in step
    if (threadIdx.x == 0) {
        s_epoch = *epoch + 1u; s_fail = 0;
        s_dead = (status != nullptr && *reinterpret_cast<volatile int32_t*>(status) != 0) ? 1 : 0;
    }
    __syncthreads();
    const uint32_t e = s_epoch;
    const bool dead = s_dead != 0;
    const uint32_t units = rows * row_units;
    for (uint32_t p = 0; p < world; ++p) {
        uint4* dst = reinterpret_cast<uint4*>(peer_bufs[p]) + (size_t)rank * slot_units;
        for (uint32_t i = threadIdx.x; i < units; i += blockDim.x) {
            const uint32_t m = i / row_units, c = i - m * row_units;
            dst[(size_t)m * pitch_units + c] = shard[i];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
        uint32_t* f = reinterpret_cast<uint32_t*>(peer_flags[threadIdx.x]) + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(e) : "memory");
        // wait for rank threadIdx.x to have pushed its slice of this exchange to me
        const uint32_t* mine = my_flags + threadIdx.x;
        unsigned long long t0 = 0;
        for (uint32_t spin = 0; !dead; ++spin) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - e) >= 0) break;
            if ((spin & 31u) == 31u) {
                if (status != nullptr && *reinterpret_cast<volatile int32_t*>(status) != 0) break;   // another waiter gave up
                unsigned long long now;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                else if (now - t0 > limit_ns) {
                    s_fail = 1;
                    if (status != nullptr) *reinterpret_cast<volatile int32_t*>(status) = 1;
                    break;
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        *epoch = e;
        if (s_fail && status != nullptr) *status = 1;
    }
}

}  // namespace mcl

using namespace mcl;

extern "C" mc_status_t mc_sm100_peer_allgather_rows(const void* d_shard, uint32_t rows, uint32_t row_bytes, uint32_t dst_pitch_bytes,
                                                    uint32_t slot_bytes, const uint64_t* d_peer_bufs, const uint64_t* d_peer_flags,
                                                    uint32_t* d_my_flags, uint32_t* d_epoch, uint32_t rank, uint32_t world,
                                                    uint64_t timeout_ns, int32_t* d_status, void* stream, int32_t pdl) {
    clear_error();
    if (d_shard == nullptr || d_peer_bufs == nullptr || d_peer_flags == nullptr || d_my_flags == nullptr ||
        d_epoch == nullptr || world == 0 || world > 64u || rank >= world || rows == 0 || (row_bytes & 15u) != 0 ||
        (slot_bytes & 15u) != 0 || (dst_pitch_bytes & 15u) != 0 || row_bytes > slot_bytes ||
        (rows > 1u && (uint64_t)rank * slot_bytes + row_bytes > dst_pitch_bytes) || !aligned16(d_shard)) {
        set_error("mc_sm100_peer_allgather: invalid args (rank=%u world=%u rows=%u row=%u slot=%u pitch=%u)", rank, world, rows,
                  row_bytes, slot_bytes, dst_pitch_bytes);
        return MC_E_INVALID_ARGUMENT;
    }
    (void)launch(peer_allgather_kernel, dim3(1), dim3(512), 0, (cudaStream_t)stream, pdl != 0, (const uint4*)d_shard, rows,
                 row_bytes / 16u, dst_pitch_bytes / 16u, slot_bytes / 16u, d_peer_bufs, d_peer_flags, d_my_flags, d_epoch, rank, world,
                 (unsigned long long)(timeout_ns ? timeout_ns : kPeerWaitDefaultNs), d_status);
    MCL_CHECK_LAUNCH("peer_allgather");
    return MC_OK;
}

extern "C" mc_status_t mc_sm100_peer_allgather(const void* d_shard, uint32_t shard_bytes, uint32_t slot_bytes,
                                               const uint64_t* d_peer_bufs, const uint64_t* d_peer_flags,
                                               uint32_t* d_my_flags, uint32_t* d_epoch, uint32_t rank, uint32_t world,
                                               uint64_t timeout_ns, int32_t* d_status, void* stream, int32_t pdl) {
    return mc_sm100_peer_allgather_rows(d_shard, 1u, shard_bytes, 0u, slot_bytes, d_peer_bufs, d_peer_flags, d_my_flags, d_epoch, rank,
                                        world, timeout_ns, d_status, stream, pdl);
}
