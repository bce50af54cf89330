// One translation unit per repetition count (compiled with -DQK_INST_R=<R>) so the
// template instantiations of the edge-statistics kernel build in parallel.
#include "qk_stats.cuh"

#ifndef QK_INST_R
#error "compile with -DQK_INST_R=<reps>"
#endif

namespace qk {
template cudaError_t launch_stats_d<QK_INST_R>(const StatsArgs&, int, cudaStream_t);
}  // namespace qk
