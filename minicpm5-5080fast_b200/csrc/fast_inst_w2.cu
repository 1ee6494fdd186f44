// Instantiations of the M = 1 decode-chain GEMV: weight bytes 2.
#include "fast_dispatch.cuh"
namespace mcl {
MCL_DEFINE_LAUNCH_FAST(2)
}  // namespace mcl
