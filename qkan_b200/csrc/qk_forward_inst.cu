// One translation unit per repetition count (compiled with -DQK_INST_R=<R>) so the
// template instantiations of the forward build in parallel.
#include "qk_forward.cuh"

#ifndef QK_INST_R
#error "compile with -DQK_INST_R=<reps>"
#endif

namespace qk {
template cudaError_t launch_fwd_d<QK_INST_R>(const FwdArgs&, bool, int, bool, cudaStream_t);
}  // namespace qk
