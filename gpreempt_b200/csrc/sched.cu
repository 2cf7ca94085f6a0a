// Workload driver and per-GPU dispatch loop.
//
// Replaces, for this path, the DISB harness the reference vendors (BenchmarkSuite,
// BenchmarkTask, Load, BasicAnalyzer: third_party/disb/src/{benchmark,load,analyzer}.cpp), the
// per-policy clients (src/cuda-clients/{gpreemptclient,blpclient}.cpp,
// src/common-clients/{baseclient,seqclient,rtonlyclient}.cpp) and the REEF scheduler thread
// (src/reef-client/reef_scheduler.cpp:246-510).
//
// One dispatcher thread per GPU owns the preempt word and every launch.  Client threads hand
// requests over through a per-client atomic state word (no mutex, no condition variable) and
// spin until it flips to DONE.  Latency-critical requests are launched the moment they are
// seen; best-effort executors are launched only while the word is clear, drain inside their
// kernels when it is raised, and are resumed from their stop point once the last
// latency-critical request has completed and every best-effort stream has quiesced.
#include "executor.h"
#include "json.h"
#include "word.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <memory>
#include <random>
#include <thread>
#include <unistd.h>

namespace gpx {

enum Policy { POLICY_BASE, POLICY_SEQ, POLICY_BLP_WAIT, POLICY_YIELD };

// ---- loads (third_party/disb/src/load.cpp) ----------------------------------------------------

struct Load {
    enum Type { Continuous, Periodic, Poisson, Trace, Burst, Dependent } type = Continuous;
    double frequency = 0;
    int priority = -1;             // the load's own priority key (config/A.json:8); -1 = not given
    uint64_t launch_delay_ns = 0;  // periodic: offset of the first launch, set by the load coordinator
    long long dropped = 0;         // arrivals given up because their successor had already arrived
    // Dependent (load.cpp:299-361): a request starts once every predecessor task has delivered its
    // result with the same serial number; the predecessors' completion counters are read here.
    std::vector<const std::atomic<uint64_t> *> prev_done;
    std::vector<std::string> prev_task_ids;
    uint64_t consumed = 0;
    std::vector<double> trace_ms;
    double on_s = 1.0, off_s = 1.0;  // burst: Poisson arrivals during `on`, silence during `off`
    long long max_requests = -1;
    uint64_t begin_ns = 0, end_ns = 0, next_ns = 0;
    uint64_t interval_ns = 0;
    size_t next_trace = 0;
    long long issued = 0;
    std::mt19937_64 rng;
    std::uniform_real_distribution<double> uni{0.0, 1.0};

    void start(uint64_t begin, uint64_t end, uint64_t seed) {
        begin_ns = begin;
        end_ns = end;
        next_ns = begin + (type == Periodic ? launch_delay_ns : 0);
        rng.seed(seed);
        if (type == Periodic && frequency > 0) interval_ns = (uint64_t)(1e9 / frequency);
        if (type == Burst) next_ns = begin + exp_interval();
    }
    uint64_t exp_interval() {
        // Exponential inter-arrival gap, load.cpp:229-237, truncated to whole microseconds.
        double u = uni(rng);
        if (u <= 0) u = 1e-12;
        double s = (-1.0 / frequency) * std::log(u);
        return (uint64_t)(s * 1e6) * 1000ull;
    }
    uint64_t burst_next(uint64_t t) {
        // Arrivals only inside the `on` part of each on+off period.
        uint64_t period = (uint64_t)((on_s + off_s) * 1e9), on = (uint64_t)(on_s * 1e9);
        uint64_t cand = t + exp_interval();
        uint64_t rel = (cand - begin_ns) % period;
        if (rel >= on) cand += period - rel;  // jump to the start of the next `on` window
        return cand;
    }
    static void sleep_until(uint64_t t) {
        for (;;) {
            uint64_t now = now_ns();
            if (now >= t) return;
            uint64_t left = t - now;
            if (left > 200000) {
                timespec ts{(time_t)((left - 100000) / 1000000000ull),
                            (long)((left - 100000) % 1000000000ull)};
                nanosleep(&ts, nullptr);
            }  // the last 200 us are spun for a precise launch time
        }
    }
    // Returns false when the run is over.  An arrival whose successor has already arrived is
    // dropped, as in the reference (load.cpp:164-176, 216-227, 279-296).
    bool wait_next(std::atomic<bool> &stop) {
        if (stop.load(std::memory_order_relaxed)) return false;
        if (max_requests >= 0 && issued >= max_requests) return false;
        uint64_t now = now_ns();
        switch (type) {
            case Continuous:
                if (now < begin_ns) sleep_until(begin_ns);
                if (now >= end_ns) return false;
                break;
            case Periodic: {
                if (frequency <= 0) return false;
                uint64_t nn = next_ns + interval_ns;
                while (nn < now) {
                    next_ns = nn;
                    nn = next_ns + interval_ns;
                    ++dropped;
                }
                if (next_ns >= end_ns) return false;
                sleep_until(next_ns);
                next_ns = nn;
                break;
            }
            case Poisson: {
                if (frequency <= 0) return false;
                uint64_t nn = next_ns + exp_interval();
                while (nn < now) {
                    next_ns = nn;
                    nn = next_ns + exp_interval();
                    ++dropped;
                }
                if (next_ns >= end_ns) return false;
                sleep_until(next_ns);
                next_ns = nn;
                break;
            }
            case Burst: {
                if (frequency <= 0) return false;
                uint64_t nn = burst_next(next_ns);
                while (nn < now) {
                    next_ns = nn;
                    nn = burst_next(next_ns);
                    ++dropped;
                }
                if (next_ns >= end_ns) return false;
                sleep_until(next_ns);
                next_ns = nn;
                break;
            }
            case Trace: {
                if (next_trace >= trace_ms.size()) return false;
                size_t nn = next_trace + 1;
                uint64_t launch = begin_ns + (uint64_t)(trace_ms[next_trace] * 1e6);
                while (nn < trace_ms.size()) {
                    uint64_t t = begin_ns + (uint64_t)(trace_ms[nn] * 1e6);
                    if (t >= now) break;
                    launch = t;
                    ++nn;
                    ++dropped;
                }
                next_trace = nn;
                if (launch >= end_ns) return false;
                sleep_until(launch);
                break;
            }
            case Dependent: {
                // every predecessor has finished request number consumed + 1
                for (;;) {
                    bool ready = !prev_done.empty();
                    for (const std::atomic<uint64_t> *c : prev_done)
                        if (c->load(std::memory_order_acquire) <= consumed) ready = false;
                    if (ready) break;
                    if (stop.load(std::memory_order_relaxed) || now_ns() >= end_ns) return false;
                    timespec ts{0, 20000};
                    nanosleep(&ts, nullptr);
                }
                ++consumed;
                if (now_ns() >= end_ns) return false;
                break;
            }
        }
        if (stop.load(std::memory_order_relaxed)) return false;
        ++issued;
        return true;
    }
};

// ---- tenants ----------------------------------------------------------------------------------

enum ReqState : int { ST_IDLE = 0, ST_HINTED, ST_SUBMITTED, ST_RUNNING, ST_SUSPENDED, ST_RESUMING, ST_DONE };

struct Record {
    uint64_t arrive, prepare, preprocess, copy_in, infer, copy_out, postprocess;  // ns
    uint64_t total() const { return prepare + preprocess + copy_in + infer + copy_out + postprocess; }
};

// What the dispatcher knows about one request source: an executor bound to a stream and a
// priority class (REEFScheduler::create_queue + bind_model_queue, include/reef_scheduler.h:67-75).
// One request is in flight per client at a time; further submissions queue behind it.
struct Client {
    int priority = 1;
    int gpu = 0;
    gpx_exec *exec = nullptr;  // null: a client without GPU work, its requests complete when seen
    cudaStream_t stream = nullptr;
    cudaEvent_t done = nullptr;
    std::atomic<int> state{ST_IDLE};
    std::atomic<uint64_t> ticket{0};
    uint64_t submit_ns = 0;
    int stop_index = -1;
    size_t resume_next = 0;   // next kernel a resume (or a windowed run) in progress has to launch
    // Windowed launching: an event after every kSegKernels launches tells the dispatcher how far
    // the GPU has got, so only a bounded number of kernels is ever queued ahead of it.
    cudaEvent_t seg_ev[8] = {};
    size_t seg_recorded = 0, seg_done = 0;
    int unlaunched_from = -1; // first kernel a cut-short resume never launched (-1: none)
    int resumes = 0;
    // Clients of the scheduler API (gpx_sched_enqueue / gpx_wait): requests are counted, not
    // queued as objects, because every request of a client runs the same executor.  `submitted`
    // is advanced by the client thread, `started` and `completed` by the dispatcher.
    bool external = false;
    std::atomic<uint64_t> submitted{0}, completed{0};
    uint64_t started = 0;
    std::atomic<int> hint{0};        // gpx_sched_hint: raise the word ahead of the next submission
    std::atomic<uint64_t> last_queue_ns{0}, last_run_ns{0};
    uint64_t launch_ns = 0;
    // schedule log: tiles run per kernel summed over the launches of one request, first kernel of
    // the launch in flight
    std::vector<long long> tiles_sum;
    int seg_from = 0;
    int log_index = -1;
    virtual ~Client() {}
};

struct Tenant : Client {
    std::string id, name, model_name;
    int batch = 1;
    int seq_len = 0;
    std::string dtype;  // "" = float32
    bool use_graph = false;
    uint64_t preprocess_us = 0;
    uint64_t seed = 0;
    Load load;
    gpx_model *model = nullptr;
    void *h_in = nullptr, *h_out = nullptr;
    // Input double buffering (best-effort tenants, `prefetch_inputs`): while a request runs, the
    // next one's input is copied, chunk by chunk, into a staging buffer on a stream of its own;
    // copyInput then is a device-to-device copy.
    void *d_stage = nullptr;
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t consumed = nullptr;  // the staging buffer has been copied into the model input
    size_t staged_off = 0;           // bytes of the next input already issued
    bool staging = false;            // a prefetch is in progress or complete
    size_t in_bytes = 0, out_bytes = 0;
    std::vector<Record> records;
    std::atomic<uint64_t> results{0};  // requests completed in the run (what dependent tasks wait for)
    Record standalone{};
    uint64_t first_ns = 0, last_ns = 0;
    cudaEvent_t ev_first = nullptr, ev_last = nullptr;
    bool ev_first_recorded = false;
};

// One line of the schedule log (config key "schedule_log"): what the dispatcher did and what the
// device-side %globaltimer trace of the executors says about it.  Host stamps are CLOCK_MONOTONIC
// ns, device stamps %globaltimer ns; the report carries the clock offset measured before and after
// the run so a reader can put both on one timeline.
struct LogEntry {
    int kind;     // 0 raise, 1 clear, 2 hp done, 3 be start, 4 be stopped, 5 be done
    int client;   // index of the tenant on its GPU list (hp or be), -1 for word events
    long long a, b, c, d;
};

struct Stats {
    std::vector<double> drain_us;      // word raised -> every best-effort stream idle (host-observed)
    std::vector<double> kernel_drain_us;  // preempted kernel: word first seen -> last CTA gone (device clock)
    std::vector<double> hp_queue_us;   // request seen by the dispatcher -> launched
    long long raises = 0;
    long long be_resumes = 0;
    long long be_launches = 0;
    std::vector<LogEntry> log;
};

// ---- dispatcher -------------------------------------------------------------------------------

struct Dispatcher {
    int device = 0;
    Policy policy = POLICY_YIELD;
    bool hint = true;
    int core = -1;  // host core of the dispatcher thread
    std::vector<Client *> hp, be;
    gpx_word *word = nullptr;
    cudaEvent_t clear_event = nullptr;
    std::atomic<bool> stop{false};
    std::atomic<bool> failed{false};
    std::thread thread;
    Stats stats;
    std::atomic_flag stats_busy = ATOMIC_FLAG_INIT;  // held for the few stores of a sample, and by readers
    std::string error;
    std::atomic<uint64_t> beat_ns{0};  // host time of the dispatcher's latest pass

    void stats_lock() {
        while (stats_busy.test_and_set(std::memory_order_acquire)) {
        }
    }
    void stats_unlock() { stats_busy.clear(std::memory_order_release); }

    bool word_raised = false;
    uint64_t t_raise = 0;
    bool drain_pending = false;
    bool schedule_log = false;
    static constexpr size_t kMaxLog = 200000;

    void log(int kind, int client, long long a = 0, long long b = 0, long long c = 0, long long d = 0) {
        if (!schedule_log || stats.log.size() >= kMaxLog) return;
        stats_lock();
        stats.log.push_back(LogEntry{kind, client, a, b, c, d});
        stats_unlock();
    }
    // Adds the tiles the kernels from `from` on ran in the launch that just ended (h_trace is current).
    void account_tiles(Client *t, size_t from) {
        if (!schedule_log || !t->exec || !t->exec->trace_on) return;
        const size_t nk = t->exec->model->kernels.size();
        if (t->tiles_sum.size() != nk) t->tiles_sum.assign(nk, 0);
        for (size_t k = from; k < nk; ++k) t->tiles_sum[k] += (long long)t->exec->h_trace[4 * k + 3];
    }

    int fail(const char *what) {
        error = std::string(what) + ": " + last_error();
        failed.store(true);
        return GPX_FAIL;
    }

    int launch_full(Client *t) {
        gpx_exec *e = t->exec;
        t->launch_ns = now_ns();
        t->last_queue_ns.store(t->launch_ns - t->submit_ns, std::memory_order_relaxed);
        if (!e) return GPX_SUCC;  // nothing to run: the request completes at the next pass
        if (e->kind == GPX_EXEC_BLP && word && word->transport == GPX_WORD_DEVICE && clear_event)
            GPX_CUDA(cudaStreamWaitEvent(t->stream, clear_event, 0));
        GPX_TRY(gpx_exec_execute(e, t->stream));
        if (e->kind == GPX_EXEC_BLP)
            GPX_CUDA(cudaMemcpyAsync(e->h_stop_index, e->d_stop_index, sizeof(int),
                                     cudaMemcpyDeviceToHost, t->stream));
        GPX_TRY(read_trace_async(t));
        GPX_CUDA(cudaEventRecord(t->done, t->stream));
        if (t->priority != 0) {
            t->seg_from = 0;
            if (schedule_log) t->tiles_sum.assign(e->model->kernels.size(), 0);
            log(3, t->log_index, (long long)now_ns(), 0);
        }
        return GPX_SUCC;
    }

    int read_trace_async(Client *t) {
        gpx_exec *e = t->exec;
        if (!e->trace_on) return GPX_SUCC;
        GPX_CUDA(cudaMemcpyAsync(e->h_trace, e->d_trace, sizeof(uint64_t) * 4 * e->model->kernels.size(),
                                 cudaMemcpyDeviceToHost, t->stream));
        return GPX_SUCC;
    }

    // Resume = re-arm the stop index and replay kernels stop..N-1 with the saved cursors
    // (BLPExecutor::resume, src/executor.cpp:280-298).  The replay is issued a few launches per
    // dispatcher pass, so a latency-critical request that arrives meanwhile is seen between
    // launches (the REEF scheduler checks its real-time queue the same way,
    // src/reef-client/reef_scheduler.cpp:498-504).
    static constexpr size_t kResumeBurst = 2;
    static constexpr size_t kSegKernels = 4;
    // Best-effort kernels queued ahead of the GPU at most (0: whole runs are enqueued at once, as
    // one graph launch).  Whatever is queued when the word goes up still has to start, see the
    // word and leave before the stream is idle again: with a whole DenseNet forward (373 kernels)
    // in the queue that took about a millisecond, during which the latency-critical kernels shared
    // the launch path with them; with a window it is a few tens of microseconds.
    size_t be_window = 16;
    // Runs of up to this many kernels are still enqueued whole (as a graph when the client asks for
    // one): their queue drains in ~0.2 ms anyway and separate launches cost ~2 % of throughput
    // (ResNet-50 b32, 61 kernels: 11.65k -> 11.40k inf/s), whereas DenseNet-201 (373 kernels) gains
    // 80-100 us of latency-critical median latency and 3 % of its own throughput from the window.
    size_t be_window_min_kernels = 64;

    // A fresh best-effort run under the window: like a resume from kernel 0 with new cursors.
    int windowed_begin(Client *t) {
        gpx_exec *e = t->exec;
        if (word && word->transport == GPX_WORD_DEVICE && clear_event)
            GPX_CUDA(cudaStreamWaitEvent(t->stream, clear_event, 0));
        GPX_TRY(exec_prologue(e, t->stream));
        t->resume_next = 0;
        t->unlaunched_from = -1;
        t->seg_recorded = t->seg_done = 0;
        t->seg_from = 0;
        if (schedule_log) t->tiles_sum.assign(e->model->kernels.size(), 0);
        log(3, t->log_index, (long long)now_ns(), 0);
        return GPX_SUCC;
    }

    int resume_begin(Client *t) {
        gpx_exec *e = t->exec;
        if (word && word->transport == GPX_WORD_DEVICE && clear_event)
            GPX_CUDA(cudaStreamWaitEvent(t->stream, clear_event, 0));
        GPX_CUDA(cudaMemcpyAsync(e->d_stop_index, e->h_minus_one, sizeof(int),
                                 cudaMemcpyHostToDevice, t->stream));
        if (e->trace_on) {
            // Fresh time stamps for the kernels that are about to be replayed, so a second
            // preemption of the same kernel is measured from its own observation of the word.
            size_t nk = e->model->kernels.size(), from = (size_t)t->stop_index;
            GPX_CUDA(cudaMemcpyAsync(e->d_trace + 4 * from, e->h_trace_init + 4 * from,
                                     sizeof(uint64_t) * 4 * (nk - from), cudaMemcpyHostToDevice, t->stream));
        }
        t->resume_next = (size_t)t->stop_index;
        t->unlaunched_from = -1;
        t->seg_recorded = t->seg_done = 0;
        t->seg_from = t->stop_index;
        log(3, t->log_index, (long long)now_ns(), t->stop_index);
        return GPX_SUCC;
    }

    int resume_finish(Client *t) {
        gpx_exec *e = t->exec;
        GPX_CUDA(cudaMemcpyAsync(e->h_stop_index, e->d_stop_index, sizeof(int),
                                 cudaMemcpyDeviceToHost, t->stream));
        GPX_TRY(read_trace_async(t));
        GPX_CUDA(cudaEventRecord(t->done, t->stream));
        return GPX_SUCC;
    }

    // Returns with the tenant RUNNING once everything is enqueued, or still RESUMING.
    int resume_continue(Client *t, bool cut_short) {
        gpx_exec *e = t->exec;
        const size_t nk = e->model->kernels.size();
        if (cut_short) {
            // The word went up again: kernels not launched yet stay unlaunched and become the
            // stop point unless an earlier kernel reports one.
            if (t->resume_next < nk) t->unlaunched_from = (int)t->resume_next;
        } else {
            const size_t max_segs = be_window / kSegKernels;
            for (size_t launched = 0; t->resume_next < nk && launched < kResumeBurst; ++launched) {
                if (max_segs) {
                    while (t->seg_done < t->seg_recorded && cudaEventQuery(t->seg_ev[t->seg_done % 8]) == cudaSuccess)
                        ++t->seg_done;
                    if (t->seg_recorded - t->seg_done >= max_segs) break;
                }
                GPX_TRY(exec_launch(e, t->resume_next, t->stream));
                ++t->resume_next;
                if (max_segs && t->resume_next % kSegKernels == 0) {
                    GPX_CUDA(cudaEventRecord(t->seg_ev[t->seg_recorded % 8], t->stream));
                    ++t->seg_recorded;
                }
            }
            if (t->resume_next < nk) return GPX_SUCC;
        }
        GPX_TRY(resume_finish(t));
        t->state.store(ST_RUNNING, std::memory_order_release);
        return GPX_SUCC;
    }

    int raise() {
        if (!word || word_raised) return GPX_SUCC;
        GPX_TRY(gpx_word_raise(word));
        word_raised = true;
        t_raise = now_ns();
        log(0, -1, (long long)t_raise);
        stats_lock();
        ++stats.raises;
        stats_unlock();
        drain_pending = false;
        for (Client *t : be)
            if (t->state.load(std::memory_order_relaxed) == ST_RUNNING ||
                t->state.load(std::memory_order_relaxed) == ST_RESUMING)
                drain_pending = true;
        return GPX_SUCC;
    }

    int clear() {
        if (!word || !word_raised) return GPX_SUCC;
        log(1, -1, (long long)now_ns());
        GPX_TRY(gpx_word_clear(word));
        if (word->transport == GPX_WORD_DEVICE) GPX_CUDA(cudaEventRecord(clear_event, word->wstream));
        word_raised = false;
        return GPX_SUCC;
    }

    // Clients of the scheduler API: the next counted request of an idle client becomes its
    // submission; a finished one is counted and the client goes back to idle.
    void admit_external(Client *t) {
        if (!t->external) return;
        int st = t->state.load(std::memory_order_acquire);
        if (st == ST_DONE) {
            t->last_run_ns.store(now_ns() - t->launch_ns, std::memory_order_relaxed);
            t->state.store(ST_IDLE, std::memory_order_relaxed);
            t->completed.fetch_add(1, std::memory_order_release);
            st = ST_IDLE;
        }
        if (st == ST_IDLE || st == ST_HINTED) {
            if (t->submitted.load(std::memory_order_acquire) > t->started) {
                ++t->started;
                t->submit_ns = now_ns();
                t->hint.store(0, std::memory_order_relaxed);
                t->state.store(ST_SUBMITTED, std::memory_order_release);
            } else if (st == ST_IDLE && t->hint.load(std::memory_order_acquire)) {
                t->state.store(ST_HINTED, std::memory_order_release);
            } else if (st == ST_HINTED && !t->hint.load(std::memory_order_acquire)) {
                t->state.store(ST_IDLE, std::memory_order_release);  // the hint was withdrawn
            }
        }
    }

    int step() {
        for (Client *t : hp) admit_external(t);
        for (Client *t : be) admit_external(t);
        // 1. latency-critical: hints raise the word early, submissions are launched at once.
        int hp_active = 0;
        bool hp_launched_this_step = false;
        for (Client *t : hp) {
            int st = t->state.load(std::memory_order_acquire);
            if (st == ST_HINTED) {
                ++hp_active;
                if (policy == POLICY_YIELD || policy == POLICY_BLP_WAIT) GPX_TRY(raise());
            } else if (st == ST_SUBMITTED) {
                ++hp_active;
                if (policy == POLICY_YIELD || policy == POLICY_BLP_WAIT) GPX_TRY(raise());
                bool may_launch = true;
                if (policy == POLICY_BLP_WAIT) {
                    // Wait-based: the latency-critical kernels are only launched once every
                    // best-effort executor has drained (blpclient.cpp:185-191).
                    for (Client *b : be)
                        if (b->state.load(std::memory_order_relaxed) == ST_RUNNING ||
                            b->state.load(std::memory_order_relaxed) == ST_RESUMING)
                            may_launch = false;
                } else if (policy == POLICY_SEQ) {
                    may_launch = seq_turn(t);
                }
                if (may_launch) {
                    stats_lock();
                    stats.hp_queue_us.push_back((now_ns() - t->submit_ns) / 1e3);
                    stats_unlock();
                    GPX_TRY(launch_full(t));
                    t->state.store(ST_RUNNING, std::memory_order_release);
                    hp_launched_this_step = true;
                }
            } else if (st == ST_RUNNING) {
                cudaError_t q = t->exec ? cudaEventQuery(t->done) : cudaSuccess;
                if (q == cudaSuccess) {
                    if (schedule_log && t->exec && t->exec->trace_on) {
                        // first CTA start and last CTA exit of the request on the device clock
                        const size_t nk = t->exec->model->kernels.size();
                        unsigned long long first = ~0ull, last = 0;
                        for (size_t k = 0; k < nk; ++k) {
                            first = std::min(first, t->exec->h_trace[4 * k + 0]);
                            last = std::max(last, t->exec->h_trace[4 * k + 1]);
                        }
                        log(2, t->log_index, (long long)first, (long long)last, (long long)t->submit_ns, (long long)t->launch_ns);
                    }
                    t->state.store(ST_DONE, std::memory_order_release);
                    seq_release(t);
                } else if (q != cudaErrorNotReady) {
                    set_error("event query failed: %s", cudaGetErrorString(q));
                    return GPX_FAIL;
                } else {
                    ++hp_active;
                }
            }
        }
        (void)hp_launched_this_step;
        // 2. best-effort progress.
        int be_running = 0;
        for (Client *t : be) {
            int st = t->state.load(std::memory_order_acquire);
            if (st == ST_RUNNING) {
                cudaError_t q = t->exec ? cudaEventQuery(t->done) : cudaSuccess;
                if (q == cudaSuccess) {
                    int stop = (t->exec && t->exec->kind == GPX_EXEC_BLP) ? *t->exec->h_stop_index : -1;
                    if (stop == -1 && t->unlaunched_from >= 0) stop = t->unlaunched_from;
                    t->unlaunched_from = -1;
                    account_tiles(t, (size_t)t->seg_from);
                    if (schedule_log && t->exec && t->exec->trace_on) {
                        const size_t nk = t->exec->model->kernels.size();
                        const unsigned long long *tr = t->exec->h_trace;
                        // first CTA start of this launch, and tiles run behind the stop point
                        unsigned long long first = ~0ull;
                        long long behind = 0;
                        for (size_t k = (size_t)t->seg_from; k < nk; ++k) first = std::min(first, tr[4 * k + 0]);
                        if (stop >= 0)
                            for (size_t k = (size_t)stop + 1; k < nk; ++k) behind += (long long)tr[4 * k + 3];
                        if (stop == -1) {
                            long long wrong = 0;
                            for (size_t k = 0; k < nk; ++k)
                                wrong += t->tiles_sum[k] != t->exec->model->kernels[k].total_tiles ? 1 : 0;
                            log(5, t->log_index, (long long)first, wrong);
                        } else {
                            log(4, t->log_index, (long long)first, stop,
                                (size_t)stop < nk ? (long long)tr[4 * (size_t)stop + 2] : -1, behind);
                        }
                    }
                    if (stop == -1) {
                        t->state.store(ST_DONE, std::memory_order_release);
                        seq_release(t);
                    } else {
                        t->stop_index = stop;
                        if (t->exec && t->exec->trace_on && (size_t)stop < t->exec->model->kernels.size()) {
                            const unsigned long long *tr = t->exec->h_trace + 4 * (size_t)stop;
                            if (tr[2] != ~0ull && tr[1] >= tr[2]) {
                                stats_lock();
                                stats.kernel_drain_us.push_back((double)(tr[1] - tr[2]) / 1e3);
                                stats_unlock();
                            }
                        }
                        t->state.store(ST_SUSPENDED, std::memory_order_release);
                    }
                } else if (q != cudaErrorNotReady) {
                    set_error("event query failed: %s", cudaGetErrorString(q));
                    return GPX_FAIL;
                } else {
                    ++be_running;
                }
            } else if (st == ST_RESUMING) {
                ++be_running;
                if (word_raised) GPX_TRY(resume_continue(t, true));
            }
        }
        if (word_raised && drain_pending && be_running == 0) {
            stats_lock();
            stats.drain_us.push_back((now_ns() - t_raise) / 1e3);
            stats_unlock();
            drain_pending = false;
        }
        // 3. the word is cleared only when no latency-critical request is in the system and
        //    every best-effort stream has quiesced, so no kernel can run ahead of an incomplete
        //    predecessor.
        if (word_raised && hp_active == 0 && be_running == 0) GPX_TRY(clear());
        // 4. best-effort launches and resumes while the word is clear.
        if (!word_raised) {
            for (Client *t : be) {
                int st = t->state.load(std::memory_order_acquire);
                if (st == ST_SUBMITTED) {
                    if (policy == POLICY_SEQ && !seq_turn(t)) continue;
                    stats_lock();
                    ++stats.be_launches;
                    stats_unlock();
                    if (be_window && t->exec && t->exec->kind == GPX_EXEC_BLP &&
                        t->exec->model->kernels.size() > be_window_min_kernels) {
                        GPX_TRY(windowed_begin(t));
                        t->state.store(ST_RESUMING, std::memory_order_release);
                        GPX_TRY(resume_continue(t, false));
                        continue;
                    }
                    GPX_TRY(launch_full(t));
                    t->state.store(ST_RUNNING, std::memory_order_release);
                } else if (st == ST_SUSPENDED) {
                    GPX_TRY(resume_begin(t));
                    stats_lock();
                    ++stats.be_resumes;
                    stats_unlock();
                    ++t->resumes;
                    t->state.store(ST_RESUMING, std::memory_order_release);
                    GPX_TRY(resume_continue(t, false));
                } else if (st == ST_RESUMING) {
                    GPX_TRY(resume_continue(t, false));
                }
            }
        }
        return GPX_SUCC;
    }

    // Strict serialisation (src/common-clients/seqclient.cpp:82-102): one request on the GPU
    // at a time, in submission order.
    Client *seq_owner = nullptr;
    bool seq_turn(Client *t) {
        if (seq_owner && seq_owner != t) return false;
        if (!seq_owner) {
            uint64_t mine = t->ticket.load(std::memory_order_relaxed);
            for (Client *o : hp)
                if (o != t && o->state.load(std::memory_order_relaxed) == ST_SUBMITTED &&
                    o->ticket.load(std::memory_order_relaxed) < mine)
                    return false;
            for (Client *o : be)
                if (o != t && o->state.load(std::memory_order_relaxed) == ST_SUBMITTED &&
                    o->ticket.load(std::memory_order_relaxed) < mine)
                    return false;
            seq_owner = t;
        }
        return true;
    }
    void seq_release(Client *t) {
        if (seq_owner == t) seq_owner = nullptr;
    }

    void run() {
        // The dispatcher gets a core of its own: when it shares one with a spinning client thread
        // the OS takes it off the CPU for whole time slices (seen as 0.7 ms dispatch delays).
        if (core >= 0) gpx_bind_core(core);
        if (gpx_init(device) != GPX_SUCC) {
            fail("dispatcher gpx_init");
            return;
        }
        while (!stop.load(std::memory_order_relaxed)) {
            if (step() != GPX_SUCC) {
                fail("dispatcher step");
                return;
            }
            beat_ns.store(now_ns(), std::memory_order_relaxed);
        }
    }
};

// ---- the benchmark suite ----------------------------------------------------------------------

static std::atomic<uint64_t> g_ticket{1};

struct Suite {
    std::vector<std::unique_ptr<Tenant>> tenants;
    std::vector<std::unique_ptr<Dispatcher>> dispatchers;  // one per GPU
    Policy policy = POLICY_YIELD;
    double time_s = 1.0;
    int warmup = 5, standalone = 20;
    uint64_t seed = 0;
    bool hint = true;
    uint64_t hint_lead_us = 0;
    bool drop_tile = false;
    size_t be_window = 16, be_window_min_kernels = 64;
    int word_transport = GPX_WORD_DEVICE;
    uint64_t request_timeout_ms = 60000;  // a request the dispatcher has not completed by then fails the run
    size_t copy_chunk = 2u << 20;  // best-effort input copies are issued in pieces of this size
    bool schedule_log = false;  // record raise / clear / start / stop events and trace every executor
    int64_t clock_off0 = 0, clock_off1 = 0, clock_unc = 0;
    uint64_t clock_t0 = 0, clock_t1 = 0;
    bool resident = false;  // inputs stay in HBM: no per-request host<->device copies
    bool prefetch_inputs = false;  // best-effort tenants stage the next input while a request runs
    std::string end_when;  // "" = time; otherwise run ends when this task hits max_requests
    std::atomic<bool> stop{false};
    uint64_t run_begin = 0, run_end = 0;

    Dispatcher *dispatcher_for(int gpu) {
        for (auto &d : dispatchers)
            if (d->device == gpu) return d.get();
        return nullptr;
    }

    // One piece of the next input into the staging buffer (one piece in flight at a time, so a
    // latency-critical input copy queues behind at most one of them).
    int stage_next_chunk(Tenant *t) {
        const size_t chunk = copy_chunk ? copy_chunk : t->in_bytes;
        const size_t nb = std::min(chunk, t->in_bytes - t->staged_off);
        GPX_CUDA(cudaMemcpyAsync((char *)t->d_stage + t->staged_off, (char *)t->h_in + t->staged_off, nb,
                                 cudaMemcpyHostToDevice, t->copy_stream));
        t->staged_off += nb;
        return GPX_SUCC;
    }

    // One request through the six phases of BenchmarkTask::inferOnce (benchmark.cpp:66-135).
    int infer_once(Tenant *t, Dispatcher *d, Record *rec) {
        uint64_t t0 = now_ns();
        rec->arrive = t0;
        uint64_t t1 = now_ns();  // prepareInput: inputs are pre-generated
        bool hinting = d->hint && t->priority == 0 && d->policy == POLICY_YIELD;
        if (t->preprocess_us) {
            // The pre-preemption hint of the reference fires SWITCH_TIME (100 us) before the
            // data-prepare phase ends (gpreemptclient.cpp:21,203-219).  Here the word is raised
            // `hint_lead_us` before the end of the phase; with the default 0 it is raised when
            // copyInput begins, which already hides the drain behind the input copy.  A longer
            // lead reserves the GPU earlier and costs the best-effort tenants that time.
            uint64_t lead = hinting ? std::min<uint64_t>(hint_lead_us, t->preprocess_us) : 0;
            usleep((useconds_t)(t->preprocess_us - lead));
            if (lead) {
                t->state.store(ST_HINTED, std::memory_order_release);
                uint64_t until = now_ns() + lead * 1000;
                while (now_ns() < until) {
                }
            }
        }
        uint64_t t2 = now_ns();
        if (hinting) t->state.store(ST_HINTED, std::memory_order_release);
        const bool prefetch = !resident && prefetch_inputs && t->priority != 0 && t->d_stage;
        if (prefetch && t->staging) {
            // finish what the wait loop of the previous request did not get to, then hand over
            while (t->staged_off < t->in_bytes) {
                GPX_CUDA(cudaStreamSynchronize(t->copy_stream));
                GPX_TRY(stage_next_chunk(t));
            }
            GPX_CUDA(cudaStreamSynchronize(t->copy_stream));
            GPX_CUDA(cudaMemcpyAsync(t->model->storages[0].dptr, t->d_stage, t->in_bytes, cudaMemcpyDeviceToDevice,
                                     t->stream));
            GPX_CUDA(cudaEventRecord(t->consumed, t->stream));
            GPX_CUDA(cudaStreamSynchronize(t->stream));
            t->staging = false;
        } else if (!resident) {
            // Best-effort inputs are copied in pieces with a synchronisation after each, so a
            // latency-critical input copy never queues behind a whole best-effort batch.
            const size_t chunk = (t->priority != 0 && copy_chunk) ? copy_chunk : t->in_bytes;
            for (size_t off = 0; off < t->in_bytes; off += chunk) {
                size_t nb = std::min(chunk, t->in_bytes - off);
                GPX_CUDA(cudaMemcpyAsync((char *)t->model->storages[0].dptr + off, (char *)t->h_in + off, nb,
                                         cudaMemcpyHostToDevice, t->stream));
                GPX_CUDA(cudaStreamSynchronize(t->stream));
            }
        }
        uint64_t t3 = now_ns();
        t->submit_ns = t3;
        t->ticket.store(g_ticket.fetch_add(1), std::memory_order_relaxed);
        t->state.store(ST_SUBMITTED, std::memory_order_release);
        if (prefetch) {
            // start staging the next request's input behind this one's hand-over
            t->staging = true;
            t->staged_off = 0;
            GPX_CUDA(cudaStreamWaitEvent(t->copy_stream, t->consumed, 0));
        }
        // Spin for the dispatcher's DONE; best-effort clients back off between polls.  The wait has a
        // deadline: a dispatcher that stopped making progress fails the request (and with it the
        // run) instead of hanging the client for ever.
        const uint64_t deadline = t3 + request_timeout_ms * 1000000ull;
        for (uint32_t spin = 0;; ++spin) {
            if (t->state.load(std::memory_order_acquire) == ST_DONE) break;
            if ((spin & 255) == 255 && now_ns() > deadline) {
                set_error("task %s: request not completed within %llu ms (dispatcher stalled?)", t->id.c_str(),
                          (unsigned long long)request_timeout_ms);
                return GPX_TIMEOUT;
            }
            if (prefetch && t->staged_off < t->in_bytes && cudaStreamQuery(t->copy_stream) == cudaSuccess)
                GPX_TRY(stage_next_chunk(t));
            if (d->failed.load(std::memory_order_relaxed)) {
                set_error("dispatcher failed: %s", d->error.c_str());
                return GPX_FAIL;
            }
            if (t->priority != 0 && (spin & 15) == 15) usleep(20);
        }
        t->state.store(ST_IDLE, std::memory_order_release);
        uint64_t t4 = now_ns();
        if (!resident && t->out_bytes) {
            int head = t->model->nodes[t->model->head_node].storage;
            GPX_CUDA(cudaMemcpyAsync(t->h_out, t->model->storages[head].dptr, t->out_bytes,
                                     cudaMemcpyDeviceToHost, t->stream));
            GPX_CUDA(cudaStreamSynchronize(t->stream));
        }
        uint64_t t5 = now_ns();
        rec->prepare = t1 - t0;
        rec->preprocess = t2 - t1;
        rec->copy_in = t3 - t2;
        rec->infer = t4 - t3;
        rec->copy_out = t5 - t4;
        rec->postprocess = 0;
        return GPX_SUCC;
    }
};

static double percentile(std::vector<double> v, double p) {
    if (v.empty()) return 0;
    std::sort(v.begin(), v.end());
    double pos = p * (v.size() - 1);
    size_t lo = (size_t)pos;
    size_t hi = std::min(lo + 1, v.size() - 1);
    return v[lo] + (v[hi] - v[lo]) * (pos - lo);
}

static Json summarize(const std::vector<double> &v) {
    Json j = Json::object();
    j.set("count", Json((long long)v.size()));
    if (v.empty()) return j;
    double sum = 0, mx = 0;
    for (double x : v) {
        sum += x;
        mx = std::max(mx, x);
    }
    j.set("mean", Json(sum / v.size()));
    j.set("p50", Json(percentile(v, 0.5)));
    j.set("p90", Json(percentile(v, 0.9)));
    j.set("p99", Json(percentile(v, 0.99)));
    j.set("max", Json(mx));
    return j;
}

static int parse_policy(const std::string &client, Policy *p, bool *rt_only, bool *hint) {
    *rt_only = false;
    *hint = true;
    if (client == "gpreemptclient" || client == "reefclient") *p = POLICY_YIELD;
    else if (client == "gpreemptclient_wo") { *p = POLICY_YIELD; *hint = false; }
    else if (client == "blpclient") *p = POLICY_BLP_WAIT;
    else if (client == "baseclient") *p = POLICY_BASE;
    else if (client == "seqclient") *p = POLICY_SEQ;
    else if (client == "rtonlyclient") { *p = POLICY_BASE; *rt_only = true; }
    else {
        set_error("unknown client '%s'", client.c_str());
        return GPX_NOT_FOUND;
    }
    return GPX_SUCC;
}

static int build_suite(Suite &s, const std::string &client, const Json &cfg) {
    bool rt_only = false, hint = true;
    GPX_TRY(parse_policy(client, &s.policy, &rt_only, &hint));
    // "reefclient": the GP policy with REEF's reset-and-restart treatment of the interrupted tile
    // (gpx_exec_set_restart_policy); the key overrides it for any client.
    s.drop_tile = cfg.has("drop_tile_in_flight") ? cfg["drop_tile_in_flight"].as_bool() : client == "reefclient";
    s.hint = cfg.has("preempt_hint") ? cfg["preempt_hint"].as_bool() : hint;
    s.hint_lead_us = (uint64_t)cfg["hint_lead_us"].as_int(0);
    s.prefetch_inputs = cfg["prefetch_inputs"].as_bool(false);
    if (cfg.has("be_window")) {
        // The window is counted in segments of kSegKernels launches tracked by a ring of eight
        // events: 0 (no window) or kSegKernels .. 8 * kSegKernels kernels.
        const long long w = cfg["be_window"].as_int(16);
        const long long lo = (long long)Dispatcher::kSegKernels, hi = 8 * lo;
        GPX_REQUIRE(w == 0 || (w >= lo && w <= hi), GPX_OUT_OF_RANGE,
                    "be_window %lld: must be 0 (whole runs are enqueued) or between %lld and %lld kernels", w, lo, hi);
        s.be_window = (size_t)w;
    }
    if (cfg.has("be_window_min_kernels")) s.be_window_min_kernels = (size_t)cfg["be_window_min_kernels"].as_int(64);
    s.time_s = cfg["time"].as_double(1.0);
    if (cfg.has("warmup")) s.warmup = (int)cfg["warmup"].as_int();
    if (cfg.has("standalone")) s.standalone = (int)cfg["standalone"].as_int();
    s.seed = (uint64_t)cfg["seed"].as_int(0);
    if (cfg.has("word_transport"))
        s.word_transport = cfg["word_transport"].as_string() == "mapped" ? GPX_WORD_MAPPED : GPX_WORD_DEVICE;
    s.end_when = cfg["end_when"].as_string();
    s.resident = cfg["resident_inputs"].as_bool(false);
    s.schedule_log = cfg["schedule_log"].as_bool(false);
    if (cfg.has("copy_chunk_bytes")) s.copy_chunk = (size_t)cfg["copy_chunk_bytes"].as_int(0);
    if (cfg.has("request_timeout_ms")) s.request_timeout_ms = (uint64_t)std::max<long long>(1, cfg["request_timeout_ms"].as_int(60000));
    int default_gpu = (int)cfg["device"].as_int(0);
    const Json &tasks = cfg["tasks"];
    GPX_REQUIRE(tasks.is_array() && tasks.size() > 0, GPX_FAIL, "config has no tasks");
    for (size_t i = 0; i < tasks.size(); ++i) {
        const Json &jt = tasks[i];
        std::string id = jt["id"].as_string();
        // rtonlyclient keeps only tasks whose id contains "_rt" (rtonlyclient.cpp:132-139).
        if (rt_only && id.find("_rt") == std::string::npos) continue;
        std::unique_ptr<Tenant> t(new Tenant());
        t->id = id;
        const Json &jc = jt["client"], &jl = jt["load"];
        t->name = jc["name"].as_string();
        t->model_name = jc["model_name"].as_string();
        // The graph-analytics tenants name their dataset beside the model (config/Z.json:
        // "model_name": "bfs", "graph_path": "crankseg_1/crankseg_1.bel").
        // Other models ignore the key, as Executor::init does (src/executor.cpp:23-45).
        if (jc.has("graph_path") && is_graph_workload(t->model_name) && t->model_name.find(':') == std::string::npos)
            t->model_name += ":" + jc["graph_path"].as_string();
        t->priority = (int)jc["priority"].as_int(1);
        t->batch = (int)jc["batch_size"].as_int(1);
        t->seq_len = (int)jc["seq_len"].as_int(0);
        if (jc.has("dtype")) t->dtype = jc["dtype"].as_string();
        t->use_graph = jc["use_cuda_graph"].as_bool(false);
        t->preprocess_us = (uint64_t)jc["preprocess_time"].as_int(0);
        t->gpu = jc.has("gpu") ? (int)jc["gpu"].as_int() : default_gpu;
        t->seed = jc.has("seed") ? (uint64_t)jc["seed"].as_int() : s.seed + 100 + i;
        std::string lt = jl["type"].as_string();
        if (lt == "continuous") t->load.type = Load::Continuous;
        else if (lt == "periodic") t->load.type = Load::Periodic;
        else if (lt == "poisson") t->load.type = Load::Poisson;
        else if (lt == "trace") t->load.type = Load::Trace;
        else if (lt == "burst") t->load.type = Load::Burst;
        else if (lt == "dependent") t->load.type = Load::Dependent;
        else {
            set_error("task %s: unknown load type '%s'", id.c_str(), lt.c_str());
            return GPX_NOT_FOUND;
        }
        t->load.frequency = jl["frequency"].as_double(0);
        if (jl.has("priority")) t->load.priority = (int)jl["priority"].as_int(0);
        if (jl.has("on")) t->load.on_s = jl["on"].as_double(1.0);
        if (jl.has("off")) t->load.off_s = jl["off"].as_double(1.0);
        if (jl.has("max_requests")) t->load.max_requests = jl["max_requests"].as_int(-1);
        const Json &prev = jl["prev_task_ids"];
        for (size_t k = 0; k < prev.size(); ++k) t->load.prev_task_ids.push_back(prev[k].as_string());
        const Json &tr = jl["trace"];
        for (size_t k = 0; k < tr.size(); ++k) t->load.trace_ms.push_back(tr[k].as_double());
        s.tenants.push_back(std::move(t));
    }
    GPX_REQUIRE(!s.tenants.empty(), GPX_FAIL, "no task left after filtering");
    for (auto &t : s.tenants) {
        if (t->load.type != Load::Dependent) continue;
        GPX_REQUIRE(!t->load.prev_task_ids.empty(), GPX_FAIL, "task %s: a dependent load needs prev_task_ids", t->id.c_str());
        for (const std::string &pid : t->load.prev_task_ids) {
            const Tenant *found = nullptr;
            for (auto &o : s.tenants)
                if (o->id == pid && o.get() != t.get()) found = o.get();
            GPX_REQUIRE(found, GPX_NOT_FOUND, "task %s depends on task '%s', which is not in the run", t->id.c_str(), pid.c_str());
            t->load.prev_done.push_back(&found->results);
        }
    }
    return GPX_SUCC;
}

static int init_tenant(Suite &s, Tenant *t) {
    GPX_TRY(gpx_init(t->gpu));
    gpx_model_opts o{};
    o.batch = t->batch;
    o.seq_len = t->seq_len;
    o.dtype = t->dtype.empty() ? nullptr : t->dtype.c_str();
    GPX_TRY(gpx_model_open(t->model_name.c_str(), &o, &t->model));
    GPX_TRY(gpx_model_init_random(t->model, 1));
    bool blp = t->priority != 0 && (s.policy == POLICY_YIELD || s.policy == POLICY_BLP_WAIT);
    GPX_TRY(gpx_exec_create(t->model, blp ? GPX_EXEC_BLP : GPX_EXEC_BASE, &t->exec));
    if (blp || s.schedule_log) GPX_TRY(gpx_exec_enable_trace(t->exec, 1));
    if (blp && s.drop_tile) GPX_TRY(gpx_exec_set_restart_policy(t->exec, 1));
    Dispatcher *d = s.dispatcher_for(t->gpu);
    if (blp) GPX_TRY(gpx_exec_set_word(t->exec, d->word));
    gpx_stream st;
    GPX_TRY(gpx_stream_create(&st, t->priority == 0 ? 0 : 1));
    t->stream = as_stream(st);
    GPX_CUDA(cudaEventCreateWithFlags(&t->done, cudaEventDisableTiming));
    for (auto &ev : t->seg_ev) GPX_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    GPX_CUDA(cudaEventCreate(&t->ev_first));
    GPX_CUDA(cudaEventCreate(&t->ev_last));
    if (t->model->sci) {
        // The scientific workload has no request data (Executor::set_input / get_output do nothing
        // for it, src/executor.cpp:47-75): a request is one time step of the resident state.
        t->in_bytes = t->out_bytes = 0;
        if (t->use_graph) GPX_TRY(gpx_exec_capture_graph(t->exec, t->stream));
        return GPX_SUCC;
    }
    const Storage &in = t->model->storages[0];
    const Storage &out = t->model->storages[t->model->nodes[t->model->head_node].storage];
    t->in_bytes = in.bytes;
    t->out_bytes = out.bytes;
    GPX_CUDA(cudaHostAlloc(&t->h_in, t->in_bytes, cudaHostAllocPortable));
    GPX_CUDA(cudaHostAlloc(&t->h_out, t->out_bytes, cudaHostAllocPortable));
    if (s.prefetch_inputs && t->priority != 0 && !s.resident) {
        GPX_CUDA(cudaMalloc(&t->d_stage, t->in_bytes));
        GPX_CUDA(cudaStreamCreateWithFlags(&t->copy_stream, cudaStreamNonBlocking));
        GPX_CUDA(cudaEventCreateWithFlags(&t->consumed, cudaEventDisableTiming));
    }
    if (in.kind == Storage::InputI64) {
        // token ids uniform over the vocabulary (rows of the word-embedding table)
        int wi = t->model->find("embeddings.word_embeddings.weight");
        double vocab = wi >= 0 ? (double)t->model->storages[wi].dims[0] : 1000.0;
        size_t n = t->in_bytes / sizeof(long long);
        std::vector<float> u(n);
        uniform_fill(u.data(), n, t->seed, 0, 0.f, 1.f);
        for (size_t i = 0; i < n; ++i) ((long long *)t->h_in)[i] = (long long)(u[i] * vocab);
    } else {
        normal_fill((float *)t->h_in, t->in_bytes / sizeof(float), t->seed, 0, 0.f, 1.f);
    }
    GPX_CUDA(cudaMemcpy(in.dptr, t->h_in, t->in_bytes, cudaMemcpyHostToDevice));
    if (t->use_graph) GPX_TRY(gpx_exec_capture_graph(t->exec, t->stream));
    return GPX_SUCC;
}

static void destroy_suite(Suite &s) {
    for (auto &d : s.dispatchers) {
        d->stop.store(true);
        if (d->thread.joinable()) d->thread.join();
    }
    for (auto &tp : s.tenants) {
        Tenant *t = tp.get();
        if (t->model) cudaSetDevice(t->gpu);
        if (t->stream) cudaStreamSynchronize(t->stream);
        if (t->exec) gpx_exec_destroy(t->exec);
        if (t->model) gpx_model_close(t->model);
        if (t->done) cudaEventDestroy(t->done);
        for (auto &ev : t->seg_ev)
            if (ev) cudaEventDestroy(ev);
        if (t->ev_first) cudaEventDestroy(t->ev_first);
        if (t->ev_last) cudaEventDestroy(t->ev_last);
        if (t->stream) cudaStreamDestroy(t->stream);
        if (t->d_stage) cudaFree(t->d_stage);
        if (t->copy_stream) cudaStreamDestroy(t->copy_stream);
        if (t->consumed) cudaEventDestroy(t->consumed);
        if (t->h_in) cudaFreeHost(t->h_in);
        if (t->h_out) cudaFreeHost(t->h_out);
    }
    for (auto &d : s.dispatchers) {
        cudaSetDevice(d->device);
        if (d->clear_event) cudaEventDestroy(d->clear_event);
        if (d->word) gpx_word_destroy(d->word);
    }
}

static int run_suite(Suite &s, Json *report) {
    // Dispatchers, one per GPU in use.
    for (auto &tp : s.tenants) {
        if (s.dispatcher_for(tp->gpu)) continue;
        std::unique_ptr<Dispatcher> d(new Dispatcher());
        d->device = tp->gpu;
        d->policy = s.policy;
        d->hint = s.hint;
        d->be_window = s.be_window;
        d->be_window_min_kernels = s.be_window_min_kernels;
        d->schedule_log = s.schedule_log;
        GPX_TRY(gpx_init(d->device));
        if (s.policy == POLICY_YIELD || s.policy == POLICY_BLP_WAIT) {
            GPX_TRY(gpx_word_create(&d->word, s.word_transport));
            GPX_CUDA(cudaEventCreateWithFlags(&d->clear_event, cudaEventDisableTiming));
            GPX_CUDA(cudaEventRecord(d->clear_event, d->word->wstream));
        }
        s.dispatchers.push_back(std::move(d));
    }
    // client->init() for every task on the calling thread (benchmark.cpp:187-199).
    for (auto &tp : s.tenants) {
        GPX_TRY(init_tenant(s, tp.get()));
        Dispatcher *d = s.dispatcher_for(tp->gpu);
        tp->log_index = (int)(tp->priority == 0 ? d->hp : d->be).size();
        (tp->priority == 0 ? d->hp : d->be).push_back(tp.get());
    }
    // Cores: dispatchers first, then one per client thread in arrival order (bind_core(cores.fetch_add(1)),
    // src/util/util.cpp:3-11); GPX_CORE_BASE moves the first one so that several processes on one
    // host do not share cores.
    const char *core_base_env = getenv("GPX_CORE_BASE");
    const int core_base = core_base_env ? atoi(core_base_env) : 0;
    // (a negative base leaves every thread to the OS scheduler: fewer cores than threads)
    for (size_t i = 0; i < s.dispatchers.size(); ++i) s.dispatchers[i]->core = core_base < 0 ? -1 : core_base + (int)i;
    for (auto &d : s.dispatchers) d->thread = std::thread([dp = d.get()] { dp->run(); });

    // Warm-up, then stand-alone latency of each client (benchmark.cpp:221-299).
    for (auto &tp : s.tenants) {
        Tenant *t = tp.get();
        GPX_TRY(gpx_init(t->gpu));
        Dispatcher *d = s.dispatcher_for(t->gpu);
        Record r{};
        for (int i = 0; i < s.warmup; ++i) GPX_TRY(s.infer_once(t, d, &r));
        Record sum{};
        int n = std::max(1, s.standalone);
        for (int i = 0; i < n; ++i) {
            GPX_TRY(s.infer_once(t, d, &r));
            sum.prepare += r.prepare;
            sum.preprocess += r.preprocess;
            sum.copy_in += r.copy_in;
            sum.infer += r.infer;
            sum.copy_out += r.copy_out;
            sum.postprocess += r.postprocess;
        }
        t->standalone.prepare = sum.prepare / n;
        t->standalone.preprocess = sum.preprocess / n;
        t->standalone.copy_in = sum.copy_in / n;
        t->standalone.infer = sum.infer / n;
        t->standalone.copy_out = sum.copy_out / n;
        t->standalone.postprocess = sum.postprocess / n;
    }
    for (auto &d : s.dispatchers) {
        d->stats = Stats();
    }
    // builtinLoadCoordinator (load.cpp:47-69): periodic latency-critical loads of equal frequency
    // are staggered by the stand-alone latencies of the ones before them, so they do not all
    // arrive at the same instant.
    {
        std::vector<std::pair<double, uint64_t>> delay_of;  // frequency -> accumulated delay
        for (auto &tp : s.tenants) {
            Tenant *t = tp.get();
            // (the load's priority key decides, as in the reference; the client's when it is absent)
            const int lp = t->load.priority >= 0 ? t->load.priority : t->priority;
            if (t->load.type != Load::Periodic || lp > 0) continue;
            size_t k = 0;
            while (k < delay_of.size() && delay_of[k].first != t->load.frequency) ++k;
            if (k == delay_of.size()) delay_of.push_back({t->load.frequency, 0});
            t->load.launch_delay_ns = delay_of[k].second;
            delay_of[k].second += t->standalone.total();
        }
    }

    if (s.schedule_log) {
        int64_t unc = 0;
        GPX_TRY(gpx_init(s.dispatchers[0]->device));
        GPX_TRY(gpx_clock_offset_ns(&s.clock_off0, &unc));
        s.clock_t0 = now_ns();
        s.clock_unc = unc;
    }
    // One thread per task (benchmark.cpp:325-328).
    s.run_begin = now_ns() + 50000000ull;
    s.run_end = s.run_begin + (uint64_t)(s.time_s * 1e9);
    std::atomic<int> core{core_base + (int)s.dispatchers.size() - 1};
    std::atomic<int> errors{0};
    std::string first_error;
    std::vector<std::thread> threads;
    for (size_t i = 0; i < s.tenants.size(); ++i) {
        Tenant *t = s.tenants[i].get();
        t->load.start(s.run_begin, s.run_end, s.seed * 7919 + 2 + i);
        t->records.reserve(1 << 16);
        threads.emplace_back([&, t] {
            if (core_base >= 0) gpx_bind_core(core.fetch_add(1) + 1);
            if (gpx_init(t->gpu) != GPX_SUCC) {
                errors.fetch_add(1);
                return;
            }
            Dispatcher *d = s.dispatcher_for(t->gpu);
            while (t->load.wait_next(s.stop)) {
                Record r{};
                if (!t->ev_first_recorded) {
                    cudaEventRecord(t->ev_first, t->stream);
                    t->ev_first_recorded = true;
                    t->first_ns = now_ns();
                }
                if (s.infer_once(t, d, &r) != GPX_SUCC) {
                    if (errors.fetch_add(1) == 0) first_error = last_error();
                    s.stop.store(true);
                    return;
                }
                t->last_ns = now_ns();
                t->records.push_back(r);
                t->results.fetch_add(1, std::memory_order_release);
            }
            cudaEventRecord(t->ev_last, t->stream);
            cudaStreamSynchronize(t->stream);
            if (!s.end_when.empty() && t->id == s.end_when) s.stop.store(true);
        });
    }
    for (auto &th : threads) th.join();
    uint64_t t_end = now_ns();
    if (s.schedule_log) {
        int64_t unc = 0;
        if (gpx_init(s.dispatchers[0]->device) == GPX_SUCC && gpx_clock_offset_ns(&s.clock_off1, &unc) == GPX_SUCC) {
            s.clock_t1 = now_ns();
            s.clock_unc = std::max<int64_t>(s.clock_unc, unc);
        }
    }
    for (auto &d : s.dispatchers) {
        d->stop.store(true);
        if (d->thread.joinable()) d->thread.join();
        if (d->failed.load()) {
            set_error("%s", d->error.c_str());
            return GPX_FAIL;
        }
    }
    if (errors.load()) {
        set_error("client thread failed: %s", first_error.c_str());
        return GPX_FAIL;
    }

    // Report: the keys of BasicAnalyzer::generateReport (analyzer.cpp:154-168) plus percentiles.
    Json root = Json::object();
    Json jt = Json::array();
    for (auto &tp : s.tenants) {
        Tenant *t = tp.get();
        Json j = Json::object();
        j.set("id", t->id);
        j.set("type", "basic");
        j.set("model", t->model_name);
        j.set("priority", Json(t->priority));
        j.set("batch_size", Json(t->batch));
        j.set("gpu", Json(t->gpu));
        size_t n = t->records.size();
        j.set("requests", Json((long long)n));
        j.set("droppedArrivals", Json(t->load.dropped));
        j.set("launchDelay(us)", Json((long long)(t->load.launch_delay_ns / 1000)));
        if (n) j.set("firstLaunchOffset(us)", Json((long long)((t->records[0].arrive - s.run_begin) / 1000)));
        double span_s = n ? (t->last_ns - s.run_begin) / 1e9 : 0;
        if (t->load.type == Load::Continuous && !s.end_when.empty() && n)
            span_s = (t->last_ns - t->first_ns) / 1e9;
        double wall_s = (std::min(t_end, s.run_end) - s.run_begin) / 1e9;
        if (!s.end_when.empty() || wall_s <= 0) wall_s = span_s;
        j.set("avgThroughput(req/s)", Json(wall_s > 0 ? n / wall_s : 0.0));
        j.set("throughput(inf/s)", Json(wall_s > 0 ? n * (double)t->batch / wall_s : 0.0));
        float dev_ms = 0;
        if (n && t->ev_first_recorded) {
            cudaSetDevice(t->gpu);
            if (cudaEventElapsedTime(&dev_ms, t->ev_first, t->ev_last) != cudaSuccess) dev_ms = 0;
        }
        j.set("deviceSpan(ms)", Json((double)dev_ms));
        Record sum{};
        std::vector<double> total_us, infer_us;
        for (const Record &r : t->records) {
            sum.prepare += r.prepare;
            sum.preprocess += r.preprocess;
            sum.copy_in += r.copy_in;
            sum.infer += r.infer;
            sum.copy_out += r.copy_out;
            sum.postprocess += r.postprocess;
            total_us.push_back(r.total() / 1e3);
            infer_us.push_back(r.infer / 1e3);
        }
        auto avg = [&](uint64_t v) { return Json((long long)(n ? v / n / 1000 : 0)); };
        long long sa = (long long)(t->standalone.total() / 1000);
        long long av = (long long)(n ? sum.total() / n / 1000 : 0);
        j.set("standAloneTotalLatency(us)", Json(sa));
        j.set("standAloneInferLatency(us)", Json((long long)(t->standalone.infer / 1000)));
        j.set("avgPrepareInputLatency(us)", avg(sum.prepare));
        j.set("avgPreprocessLatency(us)", avg(sum.preprocess));
        j.set("avgCopyInputLatency(us)", avg(sum.copy_in));
        j.set("avgInferLatency(us)", avg(sum.infer));
        j.set("avgCopyOutputLatency(us)", avg(sum.copy_out));
        j.set("avgPostprocessLatency(us)", avg(sum.postprocess));
        j.set("avgTotalLatency(us)", Json(av));
        j.set("avgTotalLatencyIncrease(us)", Json(av - sa));
        j.set("totalLatency(us)", summarize(total_us));
        j.set("inferLatency(us)", summarize(infer_us));
        j.set("resumes", Json(t->resumes));
        j.set("in_bytes", Json((long long)t->in_bytes));
        j.set("out_bytes", Json((long long)t->out_bytes));
        size_t nk = 0;
        gpx_model_kernel_num(t->model, &nk);
        j.set("kernels", Json((long long)nk));
        jt.push(j);
    }
    root.set("tasks", jt);
    Json jd = Json::array();
    for (auto &d : s.dispatchers) {
        Json j = Json::object();
        j.set("gpu", Json(d->device));
        j.set("wordRaises", Json(d->stats.raises));
        j.set("beLaunches", Json(d->stats.be_launches));
        j.set("beResumes", Json(d->stats.be_resumes));
        j.set("preemptLatency(us)", summarize(d->stats.drain_us));
        j.set("kernelDrain(us)", summarize(d->stats.kernel_drain_us));
        j.set("hpDispatchDelay(us)", summarize(d->stats.hp_queue_us));
        if (s.schedule_log) {
            // kinds: 0 raise [host ns]; 1 clear [host ns]; 2 latency-critical request done [first CTA
            // start, last CTA exit (device ns), submit, launch (host ns)]; 3 best-effort launch [host ns,
            // first kernel]; 4 best-effort launch stopped [first CTA start (device ns), stop kernel, word
            // first seen (device ns), tiles run behind the stop point]; 5 best-effort request done [first
            // CTA start of the last launch (device ns), kernels whose tiles were not run exactly once]
            // Stamps are written relative to the start of the run (host clock) and to the device
            // clock at the first offset measurement, so they stay exact as JSON numbers:
            //   host_rel = device_rel + offset_rel, with offset_rel measured before and after the run.
            const long long host_base = (long long)s.run_begin;
            const long long dev_base = (long long)s.clock_t0 - (long long)s.clock_off0;
            auto host_rel = [&](long long v) { return Json(v - host_base); };
            auto dev_rel = [&](long long v) { return (v == -1 || (unsigned long long)v == ~0ull) ? Json(-1) : Json(v - dev_base); };
            Json ev = Json::array();
            for (const LogEntry &e : d->stats.log) {
                Json r = Json::array();
                r.push(Json(e.kind));
                r.push(Json(e.client));
                switch (e.kind) {
                    case 0:
                    case 1:
                        r.push(host_rel(e.a));
                        break;
                    case 2:
                        r.push(dev_rel(e.a));
                        r.push(dev_rel(e.b));
                        r.push(host_rel(e.c));
                        r.push(host_rel(e.d));
                        break;
                    case 3:
                        r.push(host_rel(e.a));
                        r.push(Json(e.b));
                        break;
                    case 4:
                        r.push(dev_rel(e.a));
                        r.push(Json(e.b));
                        r.push(dev_rel(e.c));
                        r.push(Json(e.d));
                        break;
                    default:
                        r.push(dev_rel(e.a));
                        r.push(Json(e.b));
                        break;
                }
                ev.push(r);
            }
            Json lg = Json::object();
            lg.set("events", ev);
            lg.set("clock", "host_rel_ns = device_rel_ns + offset_rel_ns (interpolate between the two measurements)");
            lg.set("offset_before_rel_ns", Json((long long)s.clock_off0 + dev_base - host_base));
            lg.set("offset_after_rel_ns", Json((long long)s.clock_off1 + dev_base - host_base));
            lg.set("offset_before_at_rel_ns", Json((long long)s.clock_t0 - host_base));
            lg.set("offset_after_at_rel_ns", Json((long long)s.clock_t1 - host_base));
            lg.set("uncertainty_ns", Json((long long)s.clock_unc));
            j.set("scheduleLog", lg);
        }
        jd.push(j);
    }
    root.set("gpus", jd);
    root.set("elapsed(s)", Json((t_end - s.run_begin) / 1e9));
    const char *pn = s.policy == POLICY_YIELD      ? "yield"
                     : s.policy == POLICY_BLP_WAIT ? "blp-wait"
                     : s.policy == POLICY_SEQ      ? "seq"
                                                   : "base";
    root.set("policy", pn);
    root.set("preempt_hint", Json(s.hint));
    root.set("drop_tile_in_flight", Json(s.drop_tile));
    root.set("hint_lead_us", Json((int)s.hint_lead_us));
    root.set("be_window", Json((int)s.be_window));
    root.set("prefetch_inputs", Json(s.prefetch_inputs));
    root.set("resident_inputs", Json(s.resident));
    *report = root;
    return GPX_SUCC;
}

}  // namespace gpx

using namespace gpx;

static thread_local std::string g_last_report;

extern "C" int gpx_run_workload(const char *client, const char *config_json, char *report,
                                size_t cap, size_t *needed) {
    GPX_REQUIRE(client && config_json, GPX_FAIL, "NULL argument");
    Json cfg;
    std::string err;
    if (!Json::parse(config_json, &cfg, &err)) {
        set_error("config is not valid JSON: %s", err.c_str());
        return GPX_FAIL;
    }
    Suite s;
    int st = build_suite(s, client, cfg);
    Json rep;
    if (st == GPX_SUCC) st = run_suite(s, &rep);
    std::string saved = last_error();
    s.stop.store(true);
    destroy_suite(s);
    if (st != GPX_SUCC) {
        set_error("%s", saved.c_str());
        return st;
    }
    // The rendered report is kept (per calling thread) so a caller whose buffer was too small can
    // fetch it with gpx_workload_report instead of running the workload again.
    g_last_report = rep.dump(1);
    const std::string &text = g_last_report;
    if (needed) *needed = text.size() + 1;
    if (!report || cap < text.size() + 1) {
        set_error("report needs %zu bytes; fetch it with gpx_workload_report", text.size() + 1);
        return report ? GPX_OUT_OF_RANGE : GPX_SUCC;
    }
    memcpy(report, text.c_str(), text.size() + 1);
    return GPX_SUCC;
}

extern "C" int gpx_workload_report(char *report, size_t cap, size_t *needed) {
    const std::string &text = g_last_report;
    GPX_REQUIRE(!text.empty(), GPX_NOT_FOUND, "no workload has completed on this thread");
    if (needed) *needed = text.size() + 1;
    if (!report || cap < text.size() + 1) {
        set_error("report needs %zu bytes", text.size() + 1);
        return report ? GPX_OUT_OF_RANGE : GPX_SUCC;
    }
    memcpy(report, text.c_str(), text.size() + 1);
    return GPX_SUCC;
}

// ---- scheduler API ------------------------------------------------------------------------------
//
// The dispatcher behind gpx_run_workload, for clients that bring their own request loop: the
// counterpart of REEFScheduler's public interface (include/reef_scheduler.h:61-109: create_queue,
// bind_model_queue, new_task, wait_task, run, shutdown).

struct gpx_sched {
    Dispatcher d;
    std::vector<std::unique_ptr<Client>> clients;
    bool running = false;
    bool gpu_ready = false;
    std::string policy_name;
};

static int sched_gpu_setup(gpx_sched *s) {
    if (s->gpu_ready) return GPX_SUCC;
    GPX_TRY(gpx_init(s->d.device));
    if (s->d.policy == POLICY_YIELD || s->d.policy == POLICY_BLP_WAIT) {
        GPX_TRY(gpx_word_create(&s->d.word, GPX_WORD_DEVICE));
        GPX_CUDA(cudaEventCreateWithFlags(&s->d.clear_event, cudaEventDisableTiming));
        GPX_CUDA(cudaEventRecord(s->d.clear_event, s->d.word->wstream));
    }
    s->gpu_ready = true;
    return GPX_SUCC;
}

extern "C" int gpx_sched_create(int device, const char *client_policy, gpx_sched **out) {
    GPX_REQUIRE(out, GPX_FAIL, "NULL argument");
    std::unique_ptr<gpx_sched> s(new gpx_sched());
    bool rt_only = false, hint = true;
    s->policy_name = client_policy && client_policy[0] ? client_policy : "gpreemptclient";
    GPX_TRY(parse_policy(s->policy_name, &s->d.policy, &rt_only, &hint));
    s->d.device = device;
    s->d.hint = hint;
    *out = s.release();
    return GPX_SUCC;
}

extern "C" int gpx_sched_attach(gpx_sched *s, gpx_exec *exec, int priority, int *client) {
    GPX_REQUIRE(s && client, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(!s->running, GPX_FAIL, "clients are attached before gpx_sched_run");
    GPX_REQUIRE(priority == 0 || priority == 1, GPX_OUT_OF_RANGE, "priority %d: 0 = latency-critical, 1 = best-effort", priority);
    std::unique_ptr<Client> c(new Client());
    c->priority = priority;
    c->gpu = s->d.device;
    c->exec = exec;
    c->external = true;
    if (exec) {
        GPX_TRY(sched_gpu_setup(s));
        GPX_REQUIRE(exec->model->device == s->d.device, GPX_FAIL, "the executor's model lives on device %d, the scheduler on %d",
                    exec->model->device, s->d.device);
        if (exec->kind == GPX_EXEC_BLP) {
            GPX_REQUIRE(s->d.word, GPX_FAIL, "policy '%s' has no preempt word; attach a base executor", s->policy_name.c_str());
            GPX_TRY(gpx_exec_set_word(exec, s->d.word));
            GPX_TRY(gpx_exec_enable_trace(exec, 1));
        }
        gpx_stream st;
        GPX_TRY(gpx_stream_create(&st, priority == 0 ? 0 : 1));
        c->stream = as_stream(st);
        GPX_CUDA(cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming));
        for (auto &ev : c->seg_ev) GPX_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    }
    *client = (int)s->clients.size();
    (priority == 0 ? s->d.hp : s->d.be).push_back(c.get());
    s->clients.push_back(std::move(c));
    return GPX_SUCC;
}

extern "C" int gpx_sched_client_stream(gpx_sched *s, int client, gpx_stream *stream) {
    GPX_REQUIRE(s && stream, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(client >= 0 && (size_t)client < s->clients.size(), GPX_OUT_OF_RANGE, "client %d does not exist", client);
    *stream = (gpx_stream)s->clients[client]->stream;
    return GPX_SUCC;
}

extern "C" int gpx_sched_run(gpx_sched *s) {
    GPX_REQUIRE(s, GPX_FAIL, "NULL scheduler");
    GPX_REQUIRE(!s->running, GPX_FAIL, "the scheduler is already running");
    const char *core_base_env = getenv("GPX_CORE_BASE");
    s->d.core = core_base_env ? atoi(core_base_env) : -1;
    s->d.stop.store(false);
    s->d.beat_ns.store(now_ns());
    s->d.thread = std::thread([dp = &s->d] { dp->run(); });
    s->running = true;
    return GPX_SUCC;
}

extern "C" int gpx_sched_enqueue(gpx_sched *s, int client, uint64_t *ticket) {
    GPX_REQUIRE(s && ticket, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(client >= 0 && (size_t)client < s->clients.size(), GPX_OUT_OF_RANGE, "client %d does not exist", client);
    Client *c = s->clients[client].get();
    const uint64_t pending = c->submitted.load(std::memory_order_relaxed) - c->completed.load(std::memory_order_acquire);
    // (capacity of the reference's task queues, include/threadsafe_queue.h:14)
    GPX_REQUIRE(pending < 10000, GPX_FULL, "client %d has %llu requests outstanding", client, (unsigned long long)pending);
    *ticket = c->submitted.fetch_add(1, std::memory_order_release) + 1;
    return GPX_SUCC;
}

extern "C" int gpx_sched_hint(gpx_sched *s, int client, int on) {
    GPX_REQUIRE(s, GPX_FAIL, "NULL scheduler");
    GPX_REQUIRE(client >= 0 && (size_t)client < s->clients.size(), GPX_OUT_OF_RANGE, "client %d does not exist", client);
    s->clients[client]->hint.store(on ? 1 : 0, std::memory_order_release);
    return GPX_SUCC;
}

extern "C" int gpx_wait(gpx_sched *s, int client, uint64_t ticket, uint64_t timeout_ns) {
    GPX_REQUIRE(s, GPX_FAIL, "NULL scheduler");
    GPX_REQUIRE(client >= 0 && (size_t)client < s->clients.size(), GPX_OUT_OF_RANGE, "client %d does not exist", client);
    Client *c = s->clients[client].get();
    GPX_REQUIRE(ticket >= 1 && ticket <= c->submitted.load(std::memory_order_acquire), GPX_NOT_FOUND,
                "client %d has issued no ticket %llu", client, (unsigned long long)ticket);
    const uint64_t t0 = now_ns();
    for (uint32_t spin = 0;; ++spin) {
        if (c->completed.load(std::memory_order_acquire) >= ticket) return GPX_SUCC;
        if (s->d.failed.load(std::memory_order_acquire)) {
            set_error("dispatcher failed: %s", s->d.error.c_str());
            return GPX_FAIL;
        }
        if ((spin & 63) == 63) {
            if (now_ns() - t0 > timeout_ns) {
                set_error("ticket %llu of client %d not completed within %llu ns%s", (unsigned long long)ticket, client,
                          (unsigned long long)timeout_ns, s->running ? "" : " (the scheduler is not running)");
                return GPX_TIMEOUT;
            }
            if (c->priority != 0) usleep(20);
        }
    }
}

extern "C" int gpx_sched_shutdown(gpx_sched *s) {
    GPX_REQUIRE(s, GPX_FAIL, "NULL scheduler");
    if (s->running) {
        s->d.stop.store(true);
        if (s->d.thread.joinable()) s->d.thread.join();
        s->running = false;
    }
    // Whatever state the dispatcher stopped in, no kernel may find the word raised afterwards.
    if (s->d.word && s->d.word_raised) {
        gpx_word_clear(s->d.word);
        s->d.word_raised = false;
    }
    if (s->d.failed.load()) {
        set_error("dispatcher failed: %s", s->d.error.c_str());
        return GPX_FAIL;
    }
    return GPX_SUCC;
}

extern "C" int gpx_sched_destroy(gpx_sched *s) {
    if (!s) return GPX_SUCC;
    gpx_sched_shutdown(s);
    if (s->gpu_ready) cudaSetDevice(s->d.device);
    for (auto &cp : s->clients) {
        Client *c = cp.get();
        if (c->stream) cudaStreamSynchronize(c->stream);
        if (c->done) cudaEventDestroy(c->done);
        for (auto &ev : c->seg_ev)
            if (ev) cudaEventDestroy(ev);
        if (c->stream) cudaStreamDestroy(c->stream);
    }
    if (s->d.clear_event) cudaEventDestroy(s->d.clear_event);
    if (s->d.word) gpx_word_destroy(s->d.word);
    delete s;
    return GPX_SUCC;
}

extern "C" int gpx_sched_stats(gpx_sched *s, char *json, size_t cap, size_t *needed) {
    GPX_REQUIRE(s, GPX_FAIL, "NULL scheduler");
    s->d.stats_lock();
    Stats st = s->d.stats;
    s->d.stats_unlock();
    Json root = Json::object();
    root.set("policy", s->policy_name);
    root.set("running", Json(s->running));
    root.set("failed", Json(s->d.failed.load()));
    root.set("wordRaises", Json(st.raises));
    root.set("beLaunches", Json(st.be_launches));
    root.set("beResumes", Json(st.be_resumes));
    root.set("preemptLatency(us)", summarize(st.drain_us));
    root.set("kernelDrain(us)", summarize(st.kernel_drain_us));
    root.set("hpDispatchDelay(us)", summarize(st.hp_queue_us));
    Json jc = Json::array();
    for (auto &cp : s->clients) {
        Json j = Json::object();
        j.set("priority", Json(cp->priority));
        j.set("submitted", Json((long long)cp->submitted.load()));
        j.set("completed", Json((long long)cp->completed.load()));
        j.set("resumes", Json(cp->resumes));
        j.set("lastQueue(us)", Json(cp->last_queue_ns.load() / 1e3));
        j.set("lastRun(us)", Json(cp->last_run_ns.load() / 1e3));
        jc.push(j);
    }
    root.set("clients", jc);
    std::string text = root.dump(1);
    if (needed) *needed = text.size() + 1;
    if (!json || cap < text.size() + 1) {
        if (json) set_error("statistics need %zu bytes", text.size() + 1);
        return json ? GPX_OUT_OF_RANGE : GPX_SUCC;
    }
    memcpy(json, text.c_str(), text.size() + 1);
    return GPX_SUCC;
}
