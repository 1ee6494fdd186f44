// Instantiations of the M = 1 decode-chain GEMV: weight bytes 1.
#include "fast_dispatch.cuh"
namespace mcl {
MCL_DEFINE_LAUNCH_FAST(1)
}  // namespace mcl
