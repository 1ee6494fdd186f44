// Instantiations of the streaming GEMV family: weight bytes 2, math form 1.
#include "rows_dispatch.cuh"
namespace mcl {
MCL_DEFINE_LAUNCH_ROWS(2, 1)
}  // namespace mcl
