// Instantiations of the streaming GEMV family: weight bytes 1, math form 0.
#include "rows_dispatch.cuh"
namespace mcl {
MCL_DEFINE_LAUNCH_ROWS(1, 0)
}  // namespace mcl
