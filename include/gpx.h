/*
 * gpx.h — C ABI of libgpx, a B200 (sm_100a) preemptive multi-tenant inference executor.
 *
 * This is the drop-in boundary below the C++ classes of thustorage/GPreempt
 * (foo::Model, foo::Executor, foo::BaseExecutor, foo::BLPExecutor, set_priority, the DISB
 * benchmark driver).  Every entry point takes plain pointers and sizes, returns an `int`
 * status (enum gpx_status, numerically equal to the reference's `enum Status`,
 * include/util/common.h:16-23) and never terminates the process.  Each declaration cites the
 * reference interface it stands in for (paths relative to the GPreempt tree).
 *
 * Threading: handles are thread-compatible (one owner thread at a time); preempt-word
 * operations and gpx_last_error are thread-safe.
 */
#ifndef GPX_H_
#define GPX_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* include/util/common.h:16-23 (enum Status), same numeric values. */
enum gpx_status {
    GPX_SUCC = 0,
    GPX_FAIL = 1,
    GPX_TIMEOUT = 2,
    GPX_NOT_FOUND = 3,
    GPX_OUT_OF_RANGE = 4,
    GPX_FULL = 5
};

typedef struct gpx_model gpx_model; /* foo::Model, include/model.h:32-93 */
typedef struct gpx_exec gpx_exec;   /* foo::Executor / BLPExecutor, include/executor.h:14-84 */
typedef struct gpx_word gpx_word;   /* GdrEntry preempt flag, src/cuda-clients/blpclient.cpp:30-76 */
typedef void *gpx_stream;           /* GPUstream (CUstream), include/util/gpu_util.h:20 */
typedef void *gpx_event;

/* ---- runtime ------------------------------------------------------------------------ */

/* foo::util::init_cuda, src/util/gpu_util.cpp:14-25.  Binds the calling thread to `device`
 * (the reference hard-codes device 0) and retains its primary context. */
int gpx_init(int device);
int gpx_device_count(int *count);
/* Number of SMs, total HBM bytes and name of the current device. */
int gpx_device_info(int *sm_count, size_t *total_mem, char *name, size_t name_cap);
/* Text for a status code (GPUGetErrorString analogue, include/util/gpu_util.h:66-68). */
const char *gpx_strerror(int status);
/* Thread-local text of the last failure reported by this library on this thread. */
const char *gpx_last_error(void);
/* util::bind_core, src/util/util.cpp:3-11. */
int gpx_bind_core(int core_id);

/* GPUMemAlloc / GPUMemFree / GPUMemHostAlloc / GPUMemFreeHost (include/util/gpu_util.h:36-41). */
int gpx_malloc(void **dptr, size_t bytes);
int gpx_free(void *dptr);
int gpx_host_alloc(void **hptr, size_t bytes);
int gpx_host_free(void *hptr);
/* GPUMemcpyHtoDAsync / DtoHAsync / DtoDAsync (include/util/gpu_util.h:52-54).  A NULL stream
 * is the legacy default stream.  The *_sync forms block until the copy completed. */
int gpx_memcpy_h2d(void *dptr, const void *hptr, size_t bytes, gpx_stream s);
int gpx_memcpy_d2h(void *hptr, const void *dptr, size_t bytes, gpx_stream s);
int gpx_memcpy_d2d(void *dst, const void *src, size_t bytes, gpx_stream s);
int gpx_memset(void *dptr, int byte, size_t bytes, gpx_stream s);

/* GPUStreamCreateWithPriority (src/common-clients/baseclient.cpp:59-61).  `priority` uses
 * the reference's convention: 0 = latency-critical (highest CUDA priority), 1 = best-effort
 * (lowest CUDA priority). */
int gpx_stream_create(gpx_stream *s, int priority);
int gpx_stream_destroy(gpx_stream s);
int gpx_stream_sync(gpx_stream s);  /* GPUStreamSynchronize */
int gpx_stream_query(gpx_stream s); /* GPUStreamQuery: GPX_SUCC when idle, GPX_TIMEOUT when busy */
int gpx_device_sync(void);

/* CUDA events on a caller-chosen stream (device-side timing for benchmarks). */
int gpx_event_create(gpx_event *e);
int gpx_event_destroy(gpx_event e);
int gpx_event_record(gpx_event e, gpx_stream s);
int gpx_event_sync(gpx_event e);
int gpx_event_elapsed_ms(gpx_event start, gpx_event stop, float *ms);

/* set_priority(NvContext, int), include/gpreempt.h:169-173 and src/gpreempt.cpp:61-72.  The
 * reference sets the channel-group timeslice of the calling thread's context by RM ioctl
 * (1 s for priority 0, 1 us for priority 1).  Here the priority class only selects the CUDA
 * stream priority used for streams created afterwards on this thread with
 * gpx_stream_create(&s, -1); no driver setting is touched. */
int gpx_set_priority(int priority);

/* ---- preempt word ------------------------------------------------------------------- */

/* Transport of the host's store to the word the kernels poll.
 *  GPX_WORD_MAPPED : the word lives in pinned host memory mapped into the device; the host
 *                    stores to it directly (one CPU store, like the GDRCopy BAR1 store at
 *                    src/cuda-clients/blpclient.cpp:185-188) and one elected thread per CTA
 *                    polls it over PCIe.
 *  GPX_WORD_DEVICE : the word lives in HBM; the host raises/clears it with a 32-bit stream
 *                    memory operation on a dedicated highest-priority stream
 *                    (REEF's GPUWriteValue32Async, src/reef-client/reef_scheduler.cpp:320). */
enum gpx_word_transport { GPX_WORD_MAPPED = 0, GPX_WORD_DEVICE = 1 };

/* get_gdr_map, src/cuda-clients/blpclient.cpp:40-76: one shared flag word per GPU. */
int gpx_word_create(gpx_word **w, int transport);
int gpx_word_destroy(gpx_word *w);
/* `*(int*)g_stop.cpu_map = 1` / `= 0`, src/cuda-clients/blpclient.cpp:186,194. */
int gpx_word_raise(gpx_word *w);
int gpx_word_clear(gpx_word *w);
/* Device address kernels poll (BLPExecutor::dpStop, include/executor.h:75). */
int gpx_word_dptr(gpx_word *w, void **dptr);
/* Current value as the host sees it. */
int gpx_word_value(gpx_word *w, int *value);

/* ---- bounded wait kernel (pre-preemption hint) -------------------------------------- */

/* gpu_block, src/block.cu:2-4, launched by start_blocking_stream
 * (src/cuda-clients/gpreemptclient.cpp:74-77): one thread waits until *flag != 0.  Unlike the
 * reference the wait is bounded: after `timeout_ns` of %globaltimer the kernel stores
 * GPX_TIMEOUT into *status (device int) and returns; otherwise it stores GPX_SUCC. */
int gpx_block_launch(const void *flag_dptr, void *status_dptr, uint64_t timeout_ns, gpx_stream s);
/* gpu_noop, src/block.cu:6-8. */
int gpx_noop_launch(gpx_stream s);

/* ---- block-level-preemption context ------------------------------------------------- */

/* The extra kernel parameters the reference's BLP transform appends
 * (scripts/compile/convert_to_blp.py:35: preempted, pStopIndex, total_block, executed,
 * shape, kernel_id) and Model::add_block_preemption_param (src/model.cpp:366-396) binds.
 * All pointers are device addresses.  `preempted == NULL` selects the non-preemptible
 * static schedule (BaseExecutor).  `trace`, when non-NULL, points at 4 uint64 slots
 * {first CTA start, last CTA exit, first time the raised word was seen, tiles run} updated
 * with %globaltimer values. */
typedef struct gpx_blp {
    const void *preempted;
    void *stop_index;
    void *executed;
    int kernel_id;
    void *trace;
} gpx_blp;

/* ---- preemption microbenchmark kernels ---------------------------------------------- */

/* y[i] = fma(a, x[i], y[i]) over n fp32 elements with persistent CTAs that claim tiles of
 * `tile_elems` elements (0 = default) from the cursor *blp->executed and drain at a tile
 * boundary once the word is raised (scripts/compile/convert_to_blp.py:39-70).  Relaunching
 * with the same cursor resumes exactly after the last claimed tile. */
int gpx_axpy_f32(float a, const void *x, void *y, size_t n, size_t tile_elems,
                 const gpx_blp *blp, gpx_stream s);
/* Number of tiles gpx_axpy_f32 splits n elements into. */
int gpx_axpy_tiles(size_t n, size_t tile_elems, int *tiles);

/* C[M][N] (bf16) = A[M][K] (bf16, row-major) x B[N][K]^T (bf16, row-major) with fp32
 * accumulation on the tcgen05 tensor cores; persistent over all SMs; preemptible at every
 * K step: a CTA that sees the word raised spills its TMEM accumulator and {tile, k} cursor
 * to `ctx` and returns; relaunching with the same `ctx` and cursor reloads them and
 * continues in the same K order, so the result is bit-identical to an uninterrupted run.
 * `ctx` is gpx_gemm_ctx_bytes() bytes of device memory, zeroed before the first launch.
 * M, N multiples of the tile (128 x 256), K a multiple of 64. */
int gpx_gemm_bf16(const void *A, const void *B, void *C, int M, int N, int K, void *ctx,
                  const gpx_blp *blp, gpx_stream s);
int gpx_gemm_ctx_bytes(size_t *bytes);
int gpx_gemm_tiles(int M, int N, int *tiles);
/* Blocking read of the context header: *error is 0, or the code of the bounded wait that
 * gave up inside the kernel (the kernel then returned early and C is incomplete). */
int gpx_gemm_status(const void *ctx, int *error, int *error_cta);

/* Has no counterpart in the reference.  The same GEMM for callers that cannot allocate device
 * memory — a client whose device memory is handed out once by an external pool or a capped
 * container, a latency-critical thread that must stay out of the allocator (cudaMalloc may
 * synchronise the device), or code running where allocation is not permitted.  The progress
 * slots and the accumulator spill area live in a static device array inside the library
 * (8 KiB + 64 x 128 KiB = 8 396 800 bytes, held by every GPU that loads the library until the
 * process exits), so no context is passed and the call performs no cudaMalloc / cudaFree and
 * calls no allocating library routine.  Limit: at most 64 output tiles, i.e.
 * (M / 128) * (N / 256) <= 64 (for example 2048 x 1024), any K that is a multiple of 64; larger
 * products are rejected with GPX_OUT_OF_RANGE and a message naming the limit.
 *   resume = 0  start a new product: the slots and the error header are cleared on `s` first
 *               (the array keeps whatever the previous call left);
 *   resume = 1  continue a product whose previous launch drained on the preempt word.
 * The first call on a device looks up the array's device address (a one-time set-up with that
 * device current); make that first call outside any stream capture.  All calls on a device share
 * the one array: two calls whose kernels overlap on the GPU race on it, so issue them on one
 * stream or order them with events.  gpx_gemm_static_status reads the error header (blocking). */
int gpx_gemm_bf16_static(const void *A, const void *B, void *C, int M, int N, int K, int resume,
                         const gpx_blp *blp, gpx_stream s);
int gpx_gemm_static_status(int *error, int *error_cta);

/* Preemption microbenchmark: `triggers` times, launch the best-effort kernel (kind 0 = fp32
 * axpy over `size` elements, kind 1 = bf16 GEMM with M = N = K = `size`), raise the preempt
 * word after a uniformly random delay in [0, kernel time), wait for the drain, clear, resume
 * until complete, and compare the result with an uninterrupted run bit for bit.  Asserted,
 * repeated form of src/tests/test-dnn-blp.cpp:36-43.  Flag-to-drain latency = %globaltimer of
 * the last CTA exit (moved to the host clock with gpx_clock_offset_ns) minus the host time just
 * before the raise.  drain_us / seen_us (may be NULL) receive one sample per preempted launch. */
typedef struct gpx_microbench_summary {
    int triggers;     /* launches attempted */
    int preempted;    /* launches that drained before completing */
    int resumes;      /* relaunches needed to complete them */
    int mismatches;   /* runs whose result differed from the uninterrupted run (must be 0) */
    double kernel_ms; /* uninterrupted kernel time (CUDA events) */
    double drain_us_p50, drain_us_p99, drain_us_max, drain_us_mean;
    double seen_us_p50, seen_us_p99; /* raise -> first CTA observed the word */
    double clock_uncertainty_ns;
    /* Host time spent inside the raise call itself, and the longest drain counted from the call's
     * return instead of its start: a large drain_us_max with a small drain_after_return_us_max is
     * a host thread that was delayed while issuing the write, not a kernel that was slow to leave. */
    double raise_call_us_p50, raise_call_us_max;
    double drain_after_return_us_max;
    /* Launches whose first CTA started only after the word had been raised (the launch itself was
     * late): they stop at their entry check, are resumed and verified like the others, and are
     * left out of the drain statistics because no running kernel was interrupted. */
    int late_starts;
} gpx_microbench_summary;
int gpx_preempt_microbench(int kind, size_t size, int triggers, uint64_t seed, int transport,
                           double *drain_us, double *seen_us, gpx_microbench_summary *out);
/* Device-side fill with the counter-based generator (fp32, or bf16 when is_bf16) and a
 * bit-wise comparison of two device buffers; helpers of the microbenchmark and the tests. */
int gpx_fill_uniform(void *dptr, size_t n, int is_bf16, uint64_t seed, uint64_t stream, float lo,
                     float hi, gpx_stream s);
int gpx_count_diff(const void *a, const void *b, size_t bytes, uint64_t *diff, gpx_stream s);

/* ---- seeded synthetic data ---------------------------------------------------------- */

/* Counter-based generator: element i of `stream` under `seed` is a pure function of
 * (seed, stream, i).  Stands in for the constant / TVM-testing random inputs the reference
 * feeds its models (src/tests/test-dnn.cpp:25-29, scripts/compile/compile.py:66-68). */
int gpx_synth_normal(float *host, size_t n, uint64_t seed, uint64_t stream, float mean,
                     float std);
int gpx_synth_uniform(float *host, size_t n, uint64_t seed, uint64_t stream, float lo, float hi);

/* ---- model -------------------------------------------------------------------------- */

typedef struct gpx_model_opts {
    int batch;          /* client JSON key "batch_size" (config/A.json:15), default 1 */
    const char *dtype;  /* "float32" (reference), later "float16"/"bfloat16" */
    int seq_len;        /* transformer graphs only */
} gpx_model_opts;

/* Model::load_model, src/model.cpp:79-125.  `name` is a built-in graph name (resnet50, vgg16,
 * mobilenet_v2, densenet201, bert_base, ... and the reference's aliases) or a directory holding
 * mod.json + host.json (+ mod.params) in the reference's formats (src/model.cpp:128-235), as
 * gpx_model_export_dir writes them: the graph is rebuilt from the nodes of mod.json, host.json
 * must list the same functions in order (the reference's "Function name mismatch" check), and
 * the parameters are loaded when the file is there.  A mod.json written by TVM is rejected: its
 * nodes only name generated functions whose arithmetic lives in mod.cu. */
int gpx_model_open(const char *name, const gpx_model_opts *opts, gpx_model **m);
int gpx_model_close(gpx_model *m); /* Model::clear, src/model.cpp:238-260 */
/* Model::load_param, src/model.cpp:263-282; file format of ModelParamParser::parse_from_file
 * (src/model.cpp:15-55): "TVM_MODEL_PARAMS\0", u64 count, {name\0, u64 n, n x fp32}. */
int gpx_model_load_params(gpx_model *m, const char *path);
/* Writer of the same format (scripts/compile/compile.py:73-85). */
int gpx_model_save_params(gpx_model *m, const char *path);
/* Seeded synthetic weights: He-normal convolution/linear weights with batch-norm folded
 * into a bias, from a counter-based generator keyed by (seed, tensor index, element). */
int gpx_model_init_random(gpx_model *m, uint64_t seed);
/* Model::get_storage_num / get_storage_info / get_storage_size (src/model.cpp:325-345). */
int gpx_model_storage_num(gpx_model *m, size_t *n);
int gpx_model_storage_info(gpx_model *m, size_t idx, char *name, size_t name_cap,
                           size_t *bytes, char *stype, size_t stype_cap, int *is_param);
/* Model::find_storage_idx, src/model.cpp:347-356. */
int gpx_model_find(gpx_model *m, const char *name, size_t *idx);
/* Model::get / Model::set by name, src/model.cpp:288-321: whole-tensor async copies in the
 * tensor's canonical layout (activations NCHW, convolution weights OIHW, as the reference's
 * graphs use); `len < size` fails with GPX_OUT_OF_RANGE. */
int gpx_model_set(gpx_model *m, const char *name, const void *host, size_t len, gpx_stream s);
int gpx_model_get(gpx_model *m, const char *name, void *host, size_t len, gpx_stream s);
/* Shape of a storage in canonical layout; returns rank in *rank (<= 4). */
int gpx_model_shape(gpx_model *m, const char *name, int64_t dims[4], int *rank);
/* Model::get_kernel_num / get_kernel_info (src/model.cpp:323, include/model.h:22-30). */
int gpx_model_kernel_num(gpx_model *m, size_t *n);
int gpx_model_kernel_info(gpx_model *m, size_t idx, char *name, size_t name_cap,
                          uint32_t launch_params[6], int *total_tiles, double *flops,
                          double *bytes);
/* Graph description in the TVM graph-JSON shape Model::load_from_json reads
 * (src/model.cpp:128-235: nodes / arg_nodes / heads / attrs.{dltype,shape}); returns the
 * number of bytes needed (including NUL) when buf is NULL or too small. */
int gpx_model_export_json(gpx_model *m, char *buf, size_t cap, size_t *needed);
/* Writes `dir`/mod.json, host.json and mod.params: the three files the reference's model
 * directory holds (patch/tvm.patch:296-329 emits host.json: temp_args in bytes and, per fused
 * function, its kernels with launch_params[6] and argument indices; scripts/compile/compile.py:
 * 73-85 writes mod.params).  gpx_model_open(dir) loads it back. */
int gpx_model_export_dir(gpx_model *m, const char *dir);
/* The scientific workload, model name "miniweather" (3200 x 1600 cells as in
 * src/workloads/miniweather.cu:21-22; "miniweather_tiny" and "miniweather_<nx>x<nz>" are smaller
 * grids): Executor::init builds the initial state (src/executor.cpp:35-38), every execute is
 * SciCompute{Raw,Blp}::perform_timestep (src/executor.cpp:131,229), set/get of "data" are not
 * needed.  Storages "state" and "state_tmp" hold [4][nz+4][nx+4] floats in the reference's layout.
 * gpx_model_reductions is reductions(mass, te) (miniweather.cu:650-677): domain mass and total
 * energy of "state".  gpx_model_init_random puts the simulation back to its initial state. */
int gpx_model_reductions(gpx_model *m, double *mass, double *te);
/* The graph-analytics workloads, model names "bfs:<prefix>", "sssp:<prefix>", "cc:<prefix>" and
 * "pagerank:<prefix>" (Executor::init with set_graph_path, src/executor.cpp:18-34): <prefix>.col,
 * <prefix>.dst and, for sssp, <prefix>.val are the files GraphCompute*::read_graph reads
 * (src/workloads/graphcompute.cu:15-45, 345-353); a relative prefix is taken under the directory in
 * the environment variable GPX_GRAPH_BASE_PATH (the reference compiles one in, src/executor.cpp:12).
 * Every execute is one GraphCompute::compute (src/executor.cpp:129,227): the algorithm from its
 * initial state to its fixed point, from vertex 0 for bfs and sssp.  The result is the storage
 * "label" (bfs: uint32 level, 0xFFFFFFFF = not reached), "cost" (sssp: uint32 distance), "comp" (cc:
 * uint32, the smallest vertex id of the component; the reference keeps 64-bit ids) or "value"
 * (pagerank: float32).  The reference has no call that returns these or the figures below.
 * `listed_iterations` is the number of iterations in the kernel list (sized by one run when the model
 * was opened), `live_iterations` how many of them the latest run needed, `converged` is 0 if that run
 * used the whole list and still had work (pagerank: always 1, it stops after 100 iterations as
 * in graphcompute.cu:281).  Any of the output pointers may be NULL.  A graph on which an algorithm
 * needs more than 16 382 rounds (a breadth-first search that deep) is refused when it is opened;
 * the reference's host loop has no such limit. */
int gpx_model_graph_info(gpx_model *m, uint64_t *vertices, uint64_t *edges, int *listed_iterations,
                         int *live_iterations, int *converged);

/* ---- executor ----------------------------------------------------------------------- */

enum gpx_exec_kind { GPX_EXEC_BASE = 0, GPX_EXEC_BLP = 1 };

/* BaseExecutor / BLPExecutor::init (src/executor.cpp:23-45, :300-342).  A BLP executor
 * owns dpStopIndex and executed[]; the preempt word is the caller's and shared among
 * executors (include/executor.h:75). */
int gpx_exec_create(gpx_model *m, int kind, gpx_exec **e);
int gpx_exec_destroy(gpx_exec *e);
int gpx_exec_set_word(gpx_exec *e, gpx_word *w); /* blp_executor->dpStop = g_stop.d */
/* The same with a raw address, for callers that own the flag memory themselves as the reference's
 * test does (executor.dpStop = p1 with p1 from GPUMallocManaged, src/tests/test-dnn-blp.cpp:18-22):
 * any 4-byte word the device can read - device memory, or pinned host memory, which the kernels
 * then poll across the bus. */
int gpx_exec_set_word_dptr(gpx_exec *e, const void *dptr);
/* Executor::execute (src/executor.cpp:119-134) / BLPExecutor::execute (:211-232). */
int gpx_exec_execute(gpx_exec *e, gpx_stream s);
/* Executor::launch_kernel, src/executor.cpp:136-164. */
int gpx_exec_launch_kernel(gpx_exec *e, size_t idx, gpx_stream s);
/* Executor::capture_graph, src/executor.cpp:176-196. */
int gpx_exec_capture_graph(gpx_exec *e, gpx_stream s);
/* BLPExecutor::getStopPoint, src/executor.cpp:269-278: waits for the stream, returns the
 * index of the first kernel that stopped early (-1 = ran to completion) and re-arms it. */
int gpx_exec_stop_point(gpx_exec *e, gpx_stream s, int *stop_index);
/* BLPExecutor::resume, src/executor.cpp:280-298: relaunches kernels stop_index..N-1 with
 * the saved cursors.  *resumed_from receives the stop index (-1 = nothing to do). */
int gpx_exec_resume(gpx_exec *e, gpx_stream s, int *resumed_from);
/* Device %globaltimer trace of the last run: per kernel 4 uint64 (see gpx_blp.trace). */
int gpx_exec_enable_trace(gpx_exec *e, int on);
int gpx_exec_read_trace(gpx_exec *e, uint64_t *out, size_t cap_u64, size_t *n_u64);
/* Error word of the executor's tensor-core kernels (blocking read): *code is 0, or the code of
 * the bounded device wait that gave up; *where is kernel index * 1000 + CTA. */
int gpx_exec_error(gpx_exec *e, int *code, int *where);
/* Zeroes every kernel's tile cursor and progress slot on `s`, as BLPExecutor::execute does
 * before launching (src/executor.cpp:212-214); lets kernels be relaunched one by one. */
int gpx_exec_reset_cursors(gpx_exec *e, gpx_stream s);
/* What a tensor-core kernel does with the output tile it is accumulating when the word is raised.
 * 0 (default): the accumulators and the K position are saved and the tile continues after the
 * resume.  1: the tile is dropped and computed again from its first K block after the resume -
 * REEF's reset-and-restart (src/reef-client/reef_scheduler.cpp:316-357,460-510: kill the
 * best-effort kernels, restart from kernel_offset; its kernels are idempotent, as these tiles are)
 * at tile granularity: nothing is written on the way out, so the drain is shorter, at the cost of
 * repeating up to one tile of work per CTA.  Either way the result is bit-identical. */
int gpx_exec_set_restart_policy(gpx_exec *e, int drop_tile_in_flight);
/* Device address of the executed[] cursor array (one int per kernel); zeroing it re-arms every
 * kernel for a full run, as BLPExecutor::execute does (src/executor.cpp:212-214). */
int gpx_exec_cursor_dptr(gpx_exec *e, void **dptr);
/* Number of layer kernels this library has launched in this process so far (kernels replayed
 * by a CUDA graph launch are counted per graph node). */
int gpx_launch_count(uint64_t *count);
/* executed[] cursors (tiles claimed per kernel) of the last run. */
int gpx_exec_read_cursors(gpx_exec *e, int *out, size_t cap, size_t *n);

/* ---- workload driver ---------------------------------------------------------------- */

/* DISB::BenchmarkSuite::{init,run,generateReport} (third_party/disb/src/benchmark.cpp:
 * 171-354) with the client policy chosen by `client`:
 *   "blpclient"  block-level preemption (src/cuda-clients/blpclient.cpp),
 *   "baseclient" stream priorities only (src/common-clients/baseclient.cpp),
 *   "seqclient"  strict serialisation (src/common-clients/seqclient.cpp),
 *   "rtonlyclient" latency-critical tasks only (src/common-clients/rtonlyclient.cpp),
 *   "gpreemptclient" preempt word raised `preprocess_time - lead` early by a hint daemon
 *                (src/cuda-clients/gpreemptclient.cpp:203-219,267-291).
 * `config_json` follows config/A.json.  The JSON report (keys of
 * third_party/disb/src/analyzer.cpp:154-168 plus p50/p99/max and preemption latencies) is
 * written to `report`; *needed receives its length including NUL. */
int gpx_run_workload(const char *client, const char *config_json, char *report, size_t cap,
                     size_t *needed);
/* The report of the last workload this thread completed (BenchmarkSuite::generateReport can be
 * called again after run, third_party/disb/src/benchmark.cpp:340-354): when gpx_run_workload
 * returned GPX_OUT_OF_RANGE because `cap` was too small, the run is not lost; call this with a
 * buffer of *needed bytes.  NULL `report` only queries the size. */
int gpx_workload_report(char *report, size_t cap, size_t *needed);

/* ---- scheduler ---------------------------------------------------------------------- */

/* The per-GPU dispatch loop behind gpx_run_workload, for clients that bring their own request
 * loop.  Counterpart of reef::executor::REEFScheduler (include/reef_scheduler.h:61-109,
 * src/reef-client/reef_scheduler.cpp:35-260): one scheduler thread per GPU that launches
 * latency-critical requests the moment it sees them, raises the preempt word so that running
 * best-effort kernels drain, and resumes them from their stop point afterwards.  Clients talk to
 * it through per-client atomic counters (no mutex, no condition variable).
 *
 * `client_policy` is one of the names gpx_run_workload takes ("gpreemptclient", "blpclient",
 * "baseclient", "seqclient", "reefclient", ...); NULL = "gpreemptclient".  Creating a scheduler
 * touches no GPU; the first attached executor does. */
typedef struct gpx_sched gpx_sched;
int gpx_sched_create(int device, const char *client_policy, gpx_sched **s);
/* REEFScheduler::create_queue + bind_model_queue (include/reef_scheduler.h:67-75): registers an
 * executor as a request source of the given priority (0 = latency-critical: real-time queue,
 * 1 = best-effort) and returns its client index.  The scheduler creates the stream the executor
 * runs on; a BLP executor is bound to the scheduler's preempt word here, so attach it before
 * capturing its graph.  `exec` may be NULL: such a client's requests complete as soon as the
 * dispatcher sees them (dispatch-latency probe, the gpu_noop of the scheduler).  Attach every
 * client before gpx_sched_run. */
int gpx_sched_attach(gpx_sched *s, gpx_exec *exec, int priority, int *client);
/* The stream a client's executor is launched on (for input copies and graph capture). */
int gpx_sched_client_stream(gpx_sched *s, int client, gpx_stream *stream);
/* REEFScheduler::run / shutdown (include/reef_scheduler.h:101-102): start and stop the
 * dispatcher thread.  Shutdown clears the preempt word if it was left raised. */
int gpx_sched_run(gpx_sched *s);
int gpx_sched_shutdown(gpx_sched *s);
int gpx_sched_destroy(gpx_sched *s);
/* REEFScheduler::new_task (include/reef_scheduler.h:85-88): one more execution of the client's
 * executor; *ticket identifies it (1, 2, 3, ... per client).  Requests of one client run in
 * order, one at a time.  GPX_FULL when 10 000 are outstanding (the reference's queue capacity,
 * include/threadsafe_queue.h:14). */
int gpx_sched_enqueue(gpx_sched *s, int client, uint64_t *ticket);
/* REEFScheduler::wait_task (include/reef_scheduler.h:90-92), with a deadline: GPX_SUCC once the
 * request completed, GPX_TIMEOUT after `timeout_ns` (the request stays queued), GPX_FAIL when the
 * dispatcher stopped on an error. */
int gpx_wait(gpx_sched *s, int client, uint64_t ticket, uint64_t timeout_ns);
/* Pre-preemption hint (DeamonHint, src/cuda-clients/gpreemptclient.cpp:51-60,203-219): a
 * latency-critical client announces that a request is about to be submitted; the dispatcher
 * raises the preempt word now, so best-effort kernels have drained when the request arrives.
 * `on` = 0 withdraws the hint. */
int gpx_sched_hint(gpx_sched *s, int client, int on);
/* Counters and latency summaries as JSON (REEFScheduler::avg_preempt_latency,
 * include/reef_scheduler.h:104-106, and the per-GPU section of the workload report). */
int gpx_sched_stats(gpx_sched *s, char *json, size_t cap, size_t *needed);

/* Host-clock (CLOCK_MONOTONIC ns) minus device %globaltimer offset, measured by a bounded
 * ping kernel; used to place host events on the device timeline. */
int gpx_clock_offset_ns(int64_t *host_minus_device, int64_t *uncertainty_ns);
/* CLOCK_MONOTONIC in ns, the clock all host timestamps of this library use. */
uint64_t gpx_host_now_ns(void);

#ifdef __cplusplus
}
#endif
#endif /* GPX_H_ */
