// One translation unit per repetition count (compiled with -DQK_INST_R=<R>) so the
// template instantiations of the backward build in parallel.
#include "qk_backward.cuh"

#ifndef QK_INST_R
#error "compile with -DQK_INST_R=<reps>"
#endif

namespace qk {
template cudaError_t launch_bwd_d<QK_INST_R>(const BwdArgs&, bool, int, cudaStream_t);
}  // namespace qk
