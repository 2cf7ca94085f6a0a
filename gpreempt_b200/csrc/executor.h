// Executor state: the native counterpart of foo::Executor / foo::BLPExecutor
// (include/executor.h:14-84 in the reference).
#pragma once

#include "model.h"

struct gpx_exec {
    gpx_model *model = nullptr;
    int kind = GPX_EXEC_BASE;
    const int *word_dptr = nullptr;   // BLPExecutor::dpStop, owned by the caller
    int *d_stop_index = nullptr;      // BLPExecutor::dpStopIndex
    int *d_executed = nullptr;        // BLPExecutor::executed, one cursor per kernel
    unsigned long long *d_trace = nullptr;
    gpx::CgemmSlot *d_slots = nullptr;  // [kernel][kSlotsPerKernel] progress of tensor-core kernels
    float *d_partial = nullptr;         // split-K partial sums of the tensor-core kernels
    float *d_spill = nullptr;           // accumulator spill area shared by this executor's kernels
    int *d_error = nullptr;             // {code, where} written by a kernel whose bounded wait gave up
    int *h_stop_index = nullptr;      // pinned landing slot of the stop index
    int *h_minus_one = nullptr;       // pinned -1 used to re-arm the stop index
    unsigned long long *h_trace_init = nullptr;
    unsigned long long *h_trace = nullptr;  // pinned landing area for asynchronous trace read-back
    int stop_index = -1;
    bool trace_on = false;
    bool drop_tile_in_flight = false;  // restart policy of the tensor-core kernels (gpx_exec_set_restart_policy)
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
};

namespace gpx {
constexpr size_t kSlotsPerKernel = 320;  // >= the largest grid that keeps per-CTA state (2 CTAs per SM of attention)
BlpArgs exec_blp_args(gpx_exec *e, size_t idx);
int exec_launch(gpx_exec *e, size_t idx, cudaStream_t s);
// Re-arms cursors, progress slots and trace for a run from kernel 0 (what execute does first).
int exec_prologue(gpx_exec *e, cudaStream_t s);
}  // namespace gpx
