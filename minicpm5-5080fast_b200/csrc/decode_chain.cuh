// decode_chain.cuh -- interface of the one-launch M = 1 decode chain (see decode_chain.cu).
#pragma once

#include "common.cuh"

namespace mcl {

enum : uint32_t { CHAIN_IN_NONE = 0xFFFFFFFFu, CHAIN_IN_X = 0xFFFFFFFEu };
enum : uint32_t { CHAIN_BUFS = 4, CHAIN_SHAPES = 8 };

// One linear of the chain, in execution order (device table, 64 bytes).
struct ChainLinear {
    const uint8_t* w;          // [N,K] bf16 bits or e4m3 codes
    const float* scale;        // [N] row scales (e4m3) or null
    const uint16_t* norm_w;    // PRO_RESNORM: RMSNorm weights [K]
    uint32_t N, K;
    uint32_t pro, epi;         // PRO_NONE / PRO_RESNORM, EPI_STORE / EPI_SWIGLU / EPI_ARGMAX
    uint32_t in_buf;           // vector read: the activation (PRO_NONE) or the addend (PRO_RESNORM);
                               // CHAIN_IN_X: the residual starts from the step's input and nothing is added
    uint32_t out_buf;          // vector written (EPI_STORE / EPI_SWIGLU)
    uint32_t rows_per_unit;    // rows per ring slot (even behind the SwiGLU epilogue)
    uint32_t shape;            // index into ChainArgs::shape_*: linears with the same (N, rows per unit, pairing) share one
    uint64_t pad;
};
static_assert(sizeof(ChainLinear) == 64, "table entries are 64 bytes");

struct ChainArgs {
    const ChainLinear* table;
    uint32_t count;
    uint32_t H;                // residual width
    uint32_t kmax;             // largest K of the table
    uint32_t slot_bytes;       // ring slot size (multiple of 128)
    uint32_t nshapes;          // distinct (rows, granule, rows per unit) among the linears, <= CHAIN_SHAPES
    uint32_t shape_rows[CHAIN_SHAPES], shape_gran[CHAIN_SHAPES], shape_rpu[CHAIN_SHAPES];
    uint32_t* bufs[CHAIN_BUFS];   // the vectors the linears hand to one another: bf16 bits | tag << 16, one word per element
    uint32_t* arrivals;        // [count] device words, zero at creation: CTAs that have finished linear i, over all steps
    const uint16_t* x_in;      // [H] bf16, the step's input
    uint16_t* logits;          // [vocab] bf16
    float* stage_val;          // [gridDim.x] per-CTA best logit
    int32_t* stage_idx;
    int32_t* token;
    float* token_val;
    uint32_t* step;            // device word, starts at 1, advanced by the kernel
    uint32_t* ticket;          // device word, 0 between steps
    int32_t* status;           // failure word (sticky)
    uint64_t timeout_ns;
    float eps;
};

// Shared memory the kernel needs for a table whose largest inner dimension is kmax, and the slot size that
// goes with it; 0 when the shapes do not fit (the caller then runs the per-linear kernels).
uint32_t chain_slot_bytes(int wb, uint32_t H, uint32_t kmax, uint32_t max_unit_bytes);
size_t chain_smem_bytes(int wb, uint32_t H, uint32_t kmax, uint32_t slot_bytes);

// Rows per ring slot for a linear of K columns behind epilogue `epi`, for slots of slot_bytes.
uint32_t chain_rows_per_unit(int wb, uint32_t K, uint32_t epi, uint32_t slot_bytes);

// One decode step: every linear of `table` by one persistent kernel (one CTA per SM, cooperative launch).
mc_status_t decode_chain_launch(int wb, const ChainArgs& a, cudaStream_t stream);

}  // namespace mcl
