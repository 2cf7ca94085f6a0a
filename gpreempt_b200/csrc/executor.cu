// Executors: replay a model's kernel list on a stream, optionally with block-level preemption.
// Counterpart of src/executor.cpp in the reference: Executor::execute (:119-134),
// launch_kernel (:136-164), capture_graph (:176-196), BLPExecutor::execute (:211-232),
// getStopPoint (:269-278), resume (:280-298), init (:300-342).
#include "executor.h"

#include <algorithm>
#include <atomic>
#include <vector>

using namespace gpx;

namespace gpx {

std::atomic<unsigned long long> g_kernel_launches{0};

BlpArgs exec_blp_args(gpx_exec *e, size_t idx) {
    BlpArgs b{};
    const Kernel &k = e->model->kernels[idx];
    b.total_tiles = k.total_tiles;
    b.kernel_id = (int)idx;
    if (e->kind == GPX_EXEC_BLP) {
        b.preempted = e->word_dptr;
        b.stop_index = e->d_stop_index;
        b.executed = e->d_executed + idx;
    }
    if (e->trace_on) b.trace = e->d_trace + 4 * idx;
    return b;
}

int exec_launch(gpx_exec *e, size_t idx, cudaStream_t s) {
    const Kernel &k = e->model->kernels[idx];
    BlpArgs b = exec_blp_args(e, idx);
    cudaError_t err;
    if (k.type == KernelType::Cgemm) {
        // The descriptor is the model's; progress slots, spill area and error word are this
        // executor's.
        CgemmParams p = k.cgemm;
        p.slots = e->d_slots + idx * kSlotsPerKernel;
        p.spill = e->d_spill;
        p.error = e->d_error;
        if (p.k_splits > 1) p.partial = e->d_partial;
        p.drop_on_stop = e->drop_tile_in_flight ? 1 : 0;
        // The cluster reduction has no stop / resume form: preemptible executors keep the workspace
        // and the finishing kernel.
        if (e->kind != GPX_EXEC_BASE) p.cluster_reduce = 0;
        err = cgemm_launch(p, k.tile, k.grid, b, s);
    } else if (k.type == KernelType::SplitK) {
        // The convolution kernel before it has already finished the tiles (cluster reduction).
        if (k.fused_into_prev && e->kind == GPX_EXEC_BASE) return GPX_SUCC;
        SplitKParams p = k.splitk;
        p.partial = e->d_partial;
        err = splitk_launch(p, k.grid, b, s);
    } else if (k.type == KernelType::DwConv) {
        err = dwconv_launch(k.dw, k.grid, b, s);
    } else if (k.type == KernelType::LayerNorm) {
        err = layernorm_launch(k.ln, k.grid, b, s);
    } else if (k.type == KernelType::Attention) {
        err = attention_launch(k.attn, k.grid, b, s);
    } else if (k.type == KernelType::AttentionTc) {
        AttnParams p = k.attn;
        p.error = e->d_error;
        p.slots = e->kind == GPX_EXEC_BLP ? e->d_slots + idx * kSlotsPerKernel : nullptr;
        err = attention_tc_launch(p, k.grid, b, s);
    } else if (k.type == KernelType::TransposeV) {
        err = transpose_v_launch(k.attn, k.grid, b, s);
    } else if (k.type == KernelType::Im2col) {
        err = im2col_launch(k.im2col, k.grid, b, s);
    } else if (k.type == KernelType::DenseRows) {
        err = dense_rows_launch(k.dense, k.grid, b, s);
    } else if (k.type == KernelType::Stencil) {
        err = stencil_launch(k.stencil, k.grid, b, s);
    } else if (k.type == KernelType::GraphWl) {
        err = graphwl_launch(k.graphwl, k.grid, b, s);
    } else if (k.type == KernelType::ConvSimt) {
        err = conv_launch(k.conv, k.tile, k.grid, b, s);
    } else {
        err = pool_launch(k.pool, k.grid, b, s);
    }
    if (err != cudaSuccess) {
        set_error("launch of kernel %zu (%s) failed: %s", idx, k.name.c_str(),
                  cudaGetErrorString(err));
        return GPX_FAIL;
    }
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    return GPX_SUCC;
}

int exec_prologue(gpx_exec *e, cudaStream_t s) {
    size_t nk = e->model->kernels.size();
    if (e->kind == GPX_EXEC_BLP) {
        GPX_REQUIRE(e->word_dptr, GPX_FAIL, "BLP executor has no preempt word (gpx_exec_set_word)");
        // BLPExecutor::execute zeroes executed[] first (src/executor.cpp:212-214).
        GPX_CUDA(cudaMemsetAsync(e->d_executed, 0, sizeof(int) * nk, s));
        GPX_CUDA(cudaMemsetAsync(e->d_slots, 0, sizeof(CgemmSlot) * kSlotsPerKernel * nk, s));
    }
    if (e->trace_on)
        GPX_CUDA(cudaMemcpyAsync(e->d_trace, e->h_trace_init, sizeof(uint64_t) * 4 * nk,
                                 cudaMemcpyHostToDevice, s));
    return GPX_SUCC;
}

}  // namespace gpx

extern "C" {

int gpx_exec_create(gpx_model *m, int kind, gpx_exec **out) {
    GPX_REQUIRE(m && out, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(kind == GPX_EXEC_BASE || kind == GPX_EXEC_BLP, GPX_OUT_OF_RANGE,
                "unknown executor kind %d", kind);
    gpx_exec *e = new gpx_exec();
    e->model = m;
    e->kind = kind;
    size_t nk = m->kernels.size();
    // dpStopIndex and executed[] are owned by the executor (src/executor.cpp:329-333).
    GPX_CUDA(cudaMalloc((void **)&e->d_stop_index, 256));
    GPX_CUDA(cudaMalloc((void **)&e->d_executed, sizeof(int) * (nk + 1)));
    GPX_CUDA(cudaMalloc((void **)&e->d_trace, sizeof(uint64_t) * 4 * (nk + 1)));
    // Tensor-core convolutions: per-kernel progress slots, one spill area (only one kernel of an
    // executor can hold partial tiles at a time) and an error word.
    GPX_CUDA(cudaMalloc((void **)&e->d_slots, sizeof(CgemmSlot) * kSlotsPerKernel * (nk + 1)));
    GPX_CUDA(cudaMemset(e->d_slots, 0, sizeof(CgemmSlot) * kSlotsPerKernel * (nk + 1)));
    size_t spill_bytes = sizeof(float) * cgemm_spill_floats_per_cta() * (size_t)(m->max_cgemm_grid + 1);
    GPX_CUDA(cudaMalloc((void **)&e->d_spill, spill_bytes));
    GPX_CUDA(cudaMalloc((void **)&e->d_partial, sizeof(float) * (m->max_partial_floats + 64)));
    GPX_CUDA(cudaMalloc((void **)&e->d_error, 1024));
    GPX_CUDA(cudaMemset(e->d_error, 0, 1024));
    GPX_CUDA(cudaHostAlloc((void **)&e->h_stop_index, 64, cudaHostAllocPortable));
    GPX_CUDA(cudaHostAlloc((void **)&e->h_minus_one, 64, cudaHostAllocPortable));
    GPX_CUDA(cudaHostAlloc((void **)&e->h_trace_init, sizeof(uint64_t) * 4 * (nk + 1),
                           cudaHostAllocPortable));
    GPX_CUDA(cudaHostAlloc((void **)&e->h_trace, sizeof(uint64_t) * 4 * (nk + 1), cudaHostAllocPortable));
    memset(e->h_trace, 0, sizeof(uint64_t) * 4 * (nk + 1));
    *e->h_stop_index = -1;
    *e->h_minus_one = -1;
    for (size_t i = 0; i < nk + 1; ++i) {
        e->h_trace_init[4 * i + 0] = ~0ull;
        e->h_trace_init[4 * i + 1] = 0;
        e->h_trace_init[4 * i + 2] = ~0ull;
        e->h_trace_init[4 * i + 3] = 0;
    }
    GPX_CUDA(cudaMemcpy(e->d_stop_index, e->h_minus_one, sizeof(int), cudaMemcpyHostToDevice));
    GPX_CUDA(cudaMemset(e->d_executed, 0, sizeof(int) * (nk + 1)));
    GPX_CUDA(cudaMemcpy(e->d_trace, e->h_trace_init, sizeof(uint64_t) * 4 * (nk + 1),
                        cudaMemcpyHostToDevice));
    *out = e;
    return GPX_SUCC;
}

int gpx_exec_destroy(gpx_exec *e) {
    if (!e) return GPX_SUCC;
    if (e->graph_exec) cudaGraphExecDestroy(e->graph_exec);
    if (e->graph) cudaGraphDestroy(e->graph);
    cudaFree(e->d_stop_index);
    cudaFree(e->d_executed);
    cudaFree(e->d_trace);
    cudaFree(e->d_slots);
    cudaFree(e->d_spill);
    cudaFree(e->d_partial);
    cudaFree(e->d_error);
    cudaFreeHost(e->h_stop_index);
    cudaFreeHost(e->h_minus_one);
    cudaFreeHost(e->h_trace_init);
    cudaFreeHost(e->h_trace);
    delete e;
    return GPX_SUCC;
}

int gpx_exec_set_word(gpx_exec *e, gpx_word *w) {
    GPX_REQUIRE(e && w, GPX_FAIL, "NULL argument");
    void *d = nullptr;
    GPX_TRY(gpx_word_dptr(w, &d));
    GPX_REQUIRE(!e->graph_exec, GPX_FAIL, "set the preempt word before capturing the graph");
    e->word_dptr = (const int *)d;
    return GPX_SUCC;
}

int gpx_exec_set_word_dptr(gpx_exec *e, const void *dptr) {
    GPX_REQUIRE(e && dptr, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(((uintptr_t)dptr % 4) == 0, GPX_FAIL, "the preempt word must be 4-byte aligned");
    GPX_REQUIRE(!e->graph_exec || e->word_dptr == (const int *)dptr, GPX_FAIL,
                "set the preempt word before capturing the graph");
    e->word_dptr = (const int *)dptr;
    return GPX_SUCC;
}

int gpx_exec_enable_trace(gpx_exec *e, int on) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    GPX_REQUIRE(!e->graph_exec, GPX_FAIL, "enable tracing before capturing the graph");
    e->trace_on = on != 0;
    return GPX_SUCC;
}

int gpx_exec_execute(gpx_exec *e, gpx_stream stream) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    cudaStream_t s = as_stream(stream);
    if (e->graph_exec) {
        GPX_CUDA(cudaGraphLaunch(e->graph_exec, s));
        g_kernel_launches.fetch_add(e->model->kernels.size(), std::memory_order_relaxed);
        return GPX_SUCC;
    }
    GPX_TRY(exec_prologue(e, s));
    size_t nk = e->model->kernels.size();
    for (size_t i = 0; i < nk; ++i) GPX_TRY(exec_launch(e, i, s));
    return GPX_SUCC;
}

int gpx_exec_launch_kernel(gpx_exec *e, size_t idx, gpx_stream s) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    GPX_REQUIRE(idx < e->model->kernels.size(), GPX_OUT_OF_RANGE, "kernel index %zu out of range",
                idx);
    if (e->kind == GPX_EXEC_BLP)
        GPX_REQUIRE(e->word_dptr, GPX_FAIL, "BLP executor has no preempt word");
    return exec_launch(e, idx, as_stream(s));
}

int gpx_exec_capture_graph(gpx_exec *e, gpx_stream stream) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    GPX_REQUIRE(stream, GPX_FAIL, "graph capture needs a non-default stream");
    GPX_REQUIRE(!e->graph_exec, GPX_FAIL, "graph already captured");
    cudaStream_t s = as_stream(stream);
    size_t nk = e->model->kernels.size();
    // Projection shortcuts as a parallel branch (non-preemptible executors): the kernels of a
    // convolution whose only consumer takes it as its residual, and whose input also feeds the main
    // path, are captured on a second stream that forks after the block input and joins before the
    // consumer.  At batch 1 every kernel is a few CTAs, so the branch runs beside the main path
    // instead of in front of it.  A preemptible executor keeps one stream: its stop point is one
    // index into the kernel list.  The split-K workspace is one per executor, so a branch that
    // would use it while the main path does is left in line.
    std::vector<char> side(nk, 0);
    std::vector<int> join_before(nk, -1);  // kernel index -> first kernel of the branch it has to wait for
    const gpx_model &m = *e->model;
    const char *env_b = getenv("GPX_GRAPH_BRANCHES");
    if (e->kind == GPX_EXEC_BASE && !m.sci && !(env_b && env_b[0] == '0')) {
        auto uses_workspace = [&](size_t i) {
            const Kernel &k = m.kernels[i];
            return k.type == KernelType::Cgemm && k.cgemm.k_splits > 1 && !k.cgemm.cluster_reduce;
        };
        for (size_t c = 0; c < m.nodes.size(); ++c) {
            const int d = m.nodes[c].residual;
            if (d < 0 || m.nodes[d].op != Op::Conv || m.nodes[d].inputs.empty()) continue;
            int users = 0, input_users = 0;
            for (const Node &o : m.nodes) {  // consumer nodes (a residual is also listed among the inputs)
                bool uses_d = o.residual == d, uses_in = o.residual == m.nodes[d].inputs[0];
                for (int in : o.inputs) {
                    uses_d = uses_d || in == d;
                    uses_in = uses_in || in == m.nodes[d].inputs[0];
                }
                users += uses_d;
                input_users += uses_in;
            }
            if (users != 1 || input_users < 2) continue;
            // kernels of d (contiguous) and of the consumer c
            size_t b0 = nk, b1 = 0, c0 = nk;
            for (size_t i = 0; i < nk; ++i) {
                if (m.kernels[i].node == d) {
                    b0 = std::min(b0, i);
                    b1 = std::max(b1, i + 1);
                }
                if (m.kernels[i].node == (int)c) c0 = std::min(c0, i);
            }
            if (b0 >= b1 || c0 == nk || b1 > c0) continue;
            bool contiguous = true, clash = false, branch_ws = false, main_ws = false;
            for (size_t i = b0; i < b1; ++i) {
                contiguous = contiguous && m.kernels[i].node == d;
                branch_ws = branch_ws || uses_workspace(i);
            }
            for (size_t i = b1; i < c0; ++i) {
                main_ws = main_ws || uses_workspace(i);
                clash = clash || side[i] || join_before[i] >= 0;
            }
            if (!contiguous || clash || (branch_ws && main_ws) || b1 == c0) continue;
            for (size_t i = b0; i < b1; ++i) side[i] = 1;
            join_before[c0] = (int)b0;
        }
    }
    bool any_side = false;
    for (char v : side) any_side = any_side || v;
    cudaStream_t s2 = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    if (any_side) {
        GPX_CUDA(cudaStreamCreateWithFlags(&s2, cudaStreamNonBlocking));
        GPX_CUDA(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
        GPX_CUDA(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
    }
    GPX_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    int st = exec_prologue(e, s);
    cudaError_t cap = cudaSuccess;
    for (size_t i = 0; st == GPX_SUCC && cap == cudaSuccess && i < nk; ++i) {
        if (side[i] && (i == 0 || !side[i - 1])) {
            cap = cudaEventRecord(ev_fork, s);
            if (cap == cudaSuccess) cap = cudaStreamWaitEvent(s2, ev_fork, 0);
        }
        if (join_before[i] >= 0 && cap == cudaSuccess) {
            cap = cudaEventRecord(ev_join, s2);
            if (cap == cudaSuccess) cap = cudaStreamWaitEvent(s, ev_join, 0);
        }
        if (cap == cudaSuccess) st = exec_launch(e, i, side[i] ? s2 : s);
    }
    g_kernel_launches.fetch_sub(st == GPX_SUCC ? nk : 0, std::memory_order_relaxed);  // captured, not run
    cudaError_t err = cudaStreamEndCapture(s, &e->graph);
    if (s2) {
        cudaStreamDestroy(s2);
        cudaEventDestroy(ev_fork);
        cudaEventDestroy(ev_join);
    }
    if (cap != cudaSuccess) {
        set_error("graph capture with a parallel branch failed: %s", cudaGetErrorString(cap));
        return GPX_FAIL;
    }
    if (st != GPX_SUCC) return st;
    GPX_CUDA(err);
    GPX_CUDA(cudaGraphInstantiate(&e->graph_exec, e->graph, 0));
    return GPX_SUCC;
}

int gpx_exec_stop_point(gpx_exec *e, gpx_stream stream, int *stop_index) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    cudaStream_t s = as_stream(stream);
    if (e->kind != GPX_EXEC_BLP) {
        GPX_CUDA(cudaStreamSynchronize(s));
        if (stop_index) *stop_index = -1;
        return GPX_SUCC;
    }
    GPX_CUDA(cudaMemcpyAsync(e->h_stop_index, e->d_stop_index, sizeof(int),
                             cudaMemcpyDeviceToHost, s));
    GPX_CUDA(cudaStreamSynchronize(s));
    int v = *e->h_stop_index;
    if (v != -1)
        GPX_CUDA(cudaMemcpyAsync(e->d_stop_index, e->h_minus_one, sizeof(int),
                                 cudaMemcpyHostToDevice, s));
    e->stop_index = v;
    if (stop_index) *stop_index = v;
    return GPX_SUCC;
}

int gpx_exec_resume(gpx_exec *e, gpx_stream stream, int *resumed_from) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    int v = -1;
    GPX_TRY(gpx_exec_stop_point(e, stream, &v));
    if (resumed_from) *resumed_from = v;
    if (v < 0) return GPX_SUCC;
    size_t nk = e->model->kernels.size();
    GPX_REQUIRE((size_t)v < nk, GPX_FAIL, "stop index %d outside the kernel list", v);
    cudaStream_t s = as_stream(stream);
    for (size_t i = (size_t)v; i < nk; ++i) GPX_TRY(exec_launch(e, i, s));
    return GPX_SUCC;
}

int gpx_exec_error(gpx_exec *e, int *code, int *where) {
    GPX_REQUIRE(e && code, GPX_FAIL, "NULL argument");
    int h[2] = {0, 0};
    GPX_CUDA(cudaMemcpy(h, e->d_error, sizeof(h), cudaMemcpyDeviceToHost));
    *code = h[0];
    if (where) *where = h[1];
    return GPX_SUCC;
}

int gpx_exec_set_restart_policy(gpx_exec *e, int drop_tile_in_flight) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    e->drop_tile_in_flight = drop_tile_in_flight != 0;
    return GPX_SUCC;
}

int gpx_exec_reset_cursors(gpx_exec *e, gpx_stream stream) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    size_t nk = e->model->kernels.size();
    GPX_CUDA(cudaMemsetAsync(e->d_executed, 0, sizeof(int) * nk, as_stream(stream)));
    GPX_CUDA(cudaMemsetAsync(e->d_slots, 0, sizeof(CgemmSlot) * kSlotsPerKernel * nk, as_stream(stream)));
    return GPX_SUCC;
}

int gpx_exec_cursor_dptr(gpx_exec *e, void **dptr) {
    GPX_REQUIRE(e && dptr, GPX_FAIL, "NULL argument");
    *dptr = e->d_executed;
    return GPX_SUCC;
}

int gpx_launch_count(uint64_t *count) {
    GPX_REQUIRE(count, GPX_FAIL, "count is NULL");
    *count = g_kernel_launches.load(std::memory_order_relaxed);
    return GPX_SUCC;
}

int gpx_exec_read_trace(gpx_exec *e, uint64_t *out, size_t cap_u64, size_t *n_u64) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    size_t n = 4 * e->model->kernels.size();
    if (n_u64) *n_u64 = n;
    if (!out) return GPX_SUCC;
    GPX_REQUIRE(cap_u64 >= n, GPX_OUT_OF_RANGE, "trace needs %zu slots, %zu given", n, cap_u64);
    GPX_CUDA(cudaMemcpy(out, e->d_trace, n * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    return GPX_SUCC;
}

int gpx_exec_read_cursors(gpx_exec *e, int *out, size_t cap, size_t *n_out) {
    GPX_REQUIRE(e, GPX_FAIL, "NULL executor");
    size_t n = e->model->kernels.size();
    if (n_out) *n_out = n;
    if (!out) return GPX_SUCC;
    GPX_REQUIRE(cap >= n, GPX_OUT_OF_RANGE, "cursors need %zu slots, %zu given", n, cap);
    GPX_CUDA(cudaMemcpy(out, e->d_executed, n * sizeof(int), cudaMemcpyDeviceToHost));
    return GPX_SUCC;
}

}  // extern "C"
