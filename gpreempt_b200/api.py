"""Python mirror of the reference's operator interface over the libgpx C ABI.

Class and method names follow thustorage/GPreempt (include/executor.h:14-84,
include/model.h:32-93): BaseExecutor / BLPExecutor with init, set_input, get_output,
get_data_size, execute, launch_kernel, capture_graph, resume, getStopPoint, get_kernel_num,
clear.  Errors surface as GpxError carrying the reference's Status code.  Everything runs on
the GPU through libgpx; nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import binding as B
from .binding import Blp, GpxError, check  # noqa: F401

_initialised = set()


def init_cuda(device: int = 0) -> None:
    """foo::util::init_cuda (src/util/gpu_util.cpp:14-25)."""
    check(B.load().gpx_init(device))
    _initialised.add(device)


def device_sync() -> None:
    check(B.load().gpx_device_sync())


def device_info() -> dict:
    sm, mem = ctypes.c_int(), ctypes.c_size_t()
    name = ctypes.create_string_buffer(128)
    check(B.load().gpx_device_info(ctypes.byref(sm), ctypes.byref(mem), name, 128))
    return {"sm_count": sm.value, "total_mem": mem.value, "name": name.value.decode()}


class Stream:
    """GPUstream created with the reference's priority convention (0 = high, 1 = low)."""

    def __init__(self, priority: int = 1):
        self.handle = ctypes.c_void_p()
        check(B.load().gpx_stream_create(ctypes.byref(self.handle), priority))

    def sync(self) -> None:
        check(B.load().gpx_stream_sync(self.handle))

    def idle(self) -> bool:
        st = B.load().gpx_stream_query(self.handle)
        if st == B.SUCC:
            return True
        if st == B.TIMEOUT:
            return False
        check(st)
        return False

    def destroy(self) -> None:
        if self.handle:
            B.load().gpx_stream_destroy(self.handle)
            self.handle = ctypes.c_void_p()


def _h(stream) -> ctypes.c_void_p:
    if stream is None:
        return ctypes.c_void_p()
    return stream.handle if hasattr(stream, "handle") else stream


class Event:
    def __init__(self):
        self.handle = ctypes.c_void_p()
        check(B.load().gpx_event_create(ctypes.byref(self.handle)))

    def record(self, stream=None) -> None:
        check(B.load().gpx_event_record(self.handle, _h(stream)))

    def sync(self) -> None:
        check(B.load().gpx_event_sync(self.handle))

    def elapsed_ms(self, later: "Event") -> float:
        ms = ctypes.c_float()
        check(B.load().gpx_event_elapsed_ms(self.handle, later.handle, ctypes.byref(ms)))
        return ms.value

    def destroy(self) -> None:
        if self.handle:
            B.load().gpx_event_destroy(self.handle)
            self.handle = ctypes.c_void_p()


class DeviceBuffer:
    """A device allocation with numpy upload/download."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        self.ptr = ctypes.c_void_p()
        check(B.load().gpx_malloc(ctypes.byref(self.ptr), self.nbytes))

    @classmethod
    def from_numpy(cls, a: np.ndarray, stream=None) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        buf = cls(a.nbytes)
        buf.upload(a, stream)
        return buf

    def upload(self, a: np.ndarray, stream=None, offset: int = 0) -> None:
        a = np.ascontiguousarray(a)
        assert offset + a.nbytes <= self.nbytes
        check(B.load().gpx_memcpy_h2d(ctypes.c_void_p(self.ptr.value + offset),
                                       a.ctypes.data_as(ctypes.c_void_p), a.nbytes, _h(stream)))
        check(B.load().gpx_stream_sync(_h(stream)))

    def download(self, dtype, count: int | None = None, stream=None, offset: int = 0) -> np.ndarray:
        dtype = np.dtype(dtype)
        if count is None:
            count = (self.nbytes - offset) // dtype.itemsize
        out = np.empty(count, dtype)
        check(B.load().gpx_memcpy_d2h(out.ctypes.data_as(ctypes.c_void_p),
                                       ctypes.c_void_p(self.ptr.value + offset), out.nbytes,
                                       _h(stream)))
        check(B.load().gpx_stream_sync(_h(stream)))
        return out

    def zero(self, stream=None) -> None:
        check(B.load().gpx_memset(self.ptr, 0, self.nbytes, _h(stream)))
        check(B.load().gpx_stream_sync(_h(stream)))

    def free(self) -> None:
        if self.ptr:
            B.load().gpx_free(self.ptr)
            self.ptr = ctypes.c_void_p()


class PreemptWord:
    """The shared preempt flag (GdrEntry g_stop, src/cuda-clients/blpclient.cpp:30-39)."""

    def __init__(self, transport: int = B.WORD_MAPPED):
        self.handle = ctypes.c_void_p()
        check(B.load().gpx_word_create(ctypes.byref(self.handle), transport))
        d = ctypes.c_void_p()
        check(B.load().gpx_word_dptr(self.handle, ctypes.byref(d)))
        self.dptr = d

    def raise_(self) -> None:
        check(B.load().gpx_word_raise(self.handle))

    def clear(self) -> None:
        check(B.load().gpx_word_clear(self.handle))

    @property
    def value(self) -> int:
        v = ctypes.c_int()
        check(B.load().gpx_word_value(self.handle, ctypes.byref(v)))
        return v.value

    def destroy(self) -> None:
        if self.handle:
            B.load().gpx_word_destroy(self.handle)
            self.handle = ctypes.c_void_p()


class BlpContext:
    """Device-side stop index, tile cursor and trace slots for one stand-alone kernel."""

    def __init__(self, word: PreemptWord | None, kernel_id: int = 0, trace: bool = True):
        self.buf = DeviceBuffer(256)
        self.word = word
        self.kernel_id = kernel_id
        self.trace = trace
        self.reset()

    def reset(self) -> None:
        init = np.zeros(64, np.int32)
        init[0] = -1  # stop index
        init[1] = 0   # cursor
        t = init[16:32].view(np.uint64)
        t[0] = np.iinfo(np.uint64).max
        t[1] = 0
        t[2] = np.iinfo(np.uint64).max
        t[3] = 0
        self.buf.upload(init)

    def rearm(self) -> None:
        """Clears the stop index only (cursor and trace are kept), as getStopPoint does."""
        self.buf.upload(np.array([-1], np.int32))

    def struct(self) -> Blp:
        base = self.buf.ptr.value
        return Blp(self.word.dptr if self.word else None, base, base + 4, self.kernel_id,
                   base + 64 if self.trace else None)

    def read(self) -> dict:
        raw = self.buf.download(np.int32)
        t = raw[16:24].view(np.uint64)
        return {"stop_index": int(raw[0]), "cursor": int(raw[1]), "t_start": int(t[0]),
                "t_end": int(t[1]), "t_seen": int(t[2]), "tiles_run": int(t[3])}

    def free(self) -> None:
        self.buf.free()


def axpy(a: float, x: DeviceBuffer, y: DeviceBuffer, n: int, blp: BlpContext | None = None,
         stream=None, tile_elems: int = 0) -> None:
    s = blp.struct() if blp is not None else None
    check(B.load().gpx_axpy_f32(ctypes.c_float(a), x.ptr, y.ptr, n, tile_elems,
                                ctypes.byref(s) if s is not None else None, _h(stream)))


def axpy_tiles(n: int, tile_elems: int = 0) -> int:
    t = ctypes.c_int()
    check(B.load().gpx_axpy_tiles(n, tile_elems, ctypes.byref(t)))
    return t.value


class GemmContext:
    """Progress slots and accumulator spill area of the preemptible GEMM (zeroed = fresh)."""

    def __init__(self):
        n = ctypes.c_size_t()
        check(B.load().gpx_gemm_ctx_bytes(ctypes.byref(n)))
        self.buf = DeviceBuffer(n.value)
        self.buf.zero()

    def reset(self) -> None:
        self.buf.zero()

    def status(self) -> tuple[int, int]:
        err, cta = ctypes.c_int(), ctypes.c_int()
        check(B.load().gpx_gemm_status(self.buf.ptr, ctypes.byref(err), ctypes.byref(cta)))
        return err.value, cta.value

    def free(self) -> None:
        self.buf.free()


def gemm_bf16(a: DeviceBuffer, b: DeviceBuffer, c: DeviceBuffer, m: int, n: int, k: int,
              ctx: GemmContext, blp: BlpContext | None = None, stream=None) -> None:
    """C[m][n] = A[m][k] x B[n][k]^T, bf16 in/out, fp32 accumulation on tcgen05."""
    s = blp.struct() if blp is not None else None
    check(B.load().gpx_gemm_bf16(a.ptr, b.ptr, c.ptr, m, n, k, ctx.buf.ptr,
                                 ctypes.byref(s) if s is not None else None, _h(stream)))


def gemm_bf16_static(a: DeviceBuffer, b: DeviceBuffer, c: DeviceBuffer, m: int, n: int, k: int,
                     resume: bool = False, blp: BlpContext | None = None, stream=None) -> None:
    """The same GEMM with its scratch in the library's static device array: nothing is allocated
    by the call.  For callers that cannot allocate device memory; at most 64 output tiles."""
    s = blp.struct() if blp is not None else None
    check(B.load().gpx_gemm_bf16_static(a.ptr, b.ptr, c.ptr, m, n, k, int(resume),
                                        ctypes.byref(s) if s is not None else None, _h(stream)))


def gemm_static_status() -> tuple[int, int]:
    err, cta = ctypes.c_int(), ctypes.c_int()
    check(B.load().gpx_gemm_static_status(ctypes.byref(err), ctypes.byref(cta)))
    return err.value, cta.value


def gemm_tiles(m: int, n: int) -> int:
    t = ctypes.c_int()
    check(B.load().gpx_gemm_tiles(m, n, ctypes.byref(t)))
    return t.value


def synth_normal(n: int, seed: int, stream: int = 0, mean: float = 0.0, std: float = 1.0):
    out = np.empty(n, np.float32)
    check(B.load().gpx_synth_normal(out.ctypes.data_as(ctypes.c_void_p), n, seed, stream, mean, std))
    return out


def synth_uniform(n: int, seed: int, stream: int = 0, lo: float = -1.0, hi: float = 1.0):
    out = np.empty(n, np.float32)
    check(B.load().gpx_synth_uniform(out.ctypes.data_as(ctypes.c_void_p), n, seed, stream, lo, hi))
    return out


class Model:
    """foo::Model (include/model.h:32-93)."""

    def __init__(self, name: str, batch: int = 0, dtype: str = "", seq_len: int = 0):
        """`name` is a built-in graph (batch 1 and float32 unless given) or a directory holding
        mod.json + host.json (+ mod.params), whose batch and storage format are the exported ones."""
        self.handle = ctypes.c_void_p()
        opts = B.ModelOpts(batch, dtype.encode(), seq_len)
        check(B.load().gpx_model_open(name.encode(), ctypes.byref(opts), ctypes.byref(self.handle)))
        self.name = name

    def get_storage_num(self) -> int:
        n = ctypes.c_size_t()
        check(B.load().gpx_model_storage_num(self.handle, ctypes.byref(n)))
        return n.value

    def get_storage_info(self, idx: int) -> dict:
        name, stype = ctypes.create_string_buffer(256), ctypes.create_string_buffer(32)
        nbytes, is_param = ctypes.c_size_t(), ctypes.c_int()
        check(B.load().gpx_model_storage_info(self.handle, idx, name, 256, ctypes.byref(nbytes),
                                              stype, 32, ctypes.byref(is_param)))
        return {"name": name.value.decode(), "size": nbytes.value, "stype": stype.value.decode(),
                "is_param": bool(is_param.value)}

    def find_storage_idx(self, name: str) -> int:
        idx = ctypes.c_size_t()
        check(B.load().gpx_model_find(self.handle, name.encode(), ctypes.byref(idx)))
        return idx.value

    def shape(self, name: str) -> tuple:
        dims = (ctypes.c_int64 * 4)()
        rank = ctypes.c_int()
        check(B.load().gpx_model_shape(self.handle, name.encode(), dims, ctypes.byref(rank)))
        return tuple(int(dims[i]) for i in range(rank.value))

    def set(self, name: str, value: np.ndarray, stream=None) -> None:
        value = np.ascontiguousarray(value)
        check(B.load().gpx_model_set(self.handle, name.encode(),
                                     value.ctypes.data_as(ctypes.c_void_p), value.nbytes,
                                     _h(stream)))
        check(B.load().gpx_stream_sync(_h(stream)))

    def get(self, name: str, stream=None) -> np.ndarray:
        shape = self.shape(name)
        stype = self.get_storage_info(self.find_storage_idx(name))["stype"]
        out = np.empty(shape, np.uint32 if stype == "uint32" else np.float32)
        check(B.load().gpx_model_get(self.handle, name.encode(),
                                     out.ctypes.data_as(ctypes.c_void_p), out.nbytes, _h(stream)))
        check(B.load().gpx_stream_sync(_h(stream)))
        return out

    def params(self) -> dict:
        out = {}
        for i in range(self.get_storage_num()):
            info = self.get_storage_info(i)
            if info["is_param"]:
                out[info["name"]] = self.get(info["name"])
        return out

    def init_random(self, seed: int) -> None:
        check(B.load().gpx_model_init_random(self.handle, seed))

    def load_param(self, path: str) -> None:
        check(B.load().gpx_model_load_params(self.handle, path.encode()))

    def save_param(self, path: str) -> None:
        check(B.load().gpx_model_save_params(self.handle, path.encode()))

    def get_kernel_num(self) -> int:
        n = ctypes.c_size_t()
        check(B.load().gpx_model_kernel_num(self.handle, ctypes.byref(n)))
        return n.value

    def get_kernel_info(self, idx: int) -> dict:
        name = ctypes.create_string_buffer(256)
        lp = (ctypes.c_uint32 * 6)()
        tiles, flops, nbytes = ctypes.c_int(), ctypes.c_double(), ctypes.c_double()
        check(B.load().gpx_model_kernel_info(self.handle, idx, name, 256, lp, ctypes.byref(tiles),
                                             ctypes.byref(flops), ctypes.byref(nbytes)))
        return {"name": name.value.decode(), "launch_params": list(lp), "total_tiles": tiles.value,
                "flops": flops.value, "bytes": nbytes.value}

    def export_json(self) -> str:
        need = ctypes.c_size_t()
        check(B.load().gpx_model_export_json(self.handle, None, 0, ctypes.byref(need)))
        buf = ctypes.create_string_buffer(need.value)
        check(B.load().gpx_model_export_json(self.handle, buf, need.value, ctypes.byref(need)))
        return buf.value.decode()

    def export_dir(self, path: str) -> None:
        """Writes mod.json, host.json and mod.params into `path`; Model(path) loads them back."""
        check(B.load().gpx_model_export_dir(self.handle, path.encode()))

    def reductions(self) -> tuple[float, float]:
        """Domain mass and total energy of a miniweather model's state
        (reductions, src/workloads/miniweather.cu:650-677)."""
        mass, te = ctypes.c_double(), ctypes.c_double()
        check(B.load().gpx_model_reductions(self.handle, ctypes.byref(mass), ctypes.byref(te)))
        return mass.value, te.value

    def graph_info(self) -> dict:
        """Sizes and iteration counts of a graph-analytics model ("bfs:<prefix>", "sssp:...",
        "cc:...", "pagerank:..."; the workloads of src/workloads/graphcompute.cu)."""
        v, e = ctypes.c_uint64(), ctypes.c_uint64()
        listed, live, conv = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        check(B.load().gpx_model_graph_info(self.handle, ctypes.byref(v), ctypes.byref(e), ctypes.byref(listed),
                                            ctypes.byref(live), ctypes.byref(conv)))
        return {"vertices": v.value, "edges": e.value, "listed_iterations": listed.value,
                "live_iterations": live.value, "converged": bool(conv.value)}

    def clear(self) -> None:
        if self.handle:
            B.load().gpx_model_close(self.handle)
            self.handle = ctypes.c_void_p()


class Executor:
    """foo::Executor (include/executor.h:14-49)."""

    KIND = B.EXEC_BASE

    def __init__(self):
        self.model: Model | None = None
        self.handle = ctypes.c_void_p()
        self.batch = 1
        self.dtype = "float32"
        self.graph_path = ""

    def set_graph_path(self, path: str) -> None:
        """Executor::set_graph_path (src/executor.cpp:18-21): the dataset of "cc", "bfs", "pagerank"
        and "sssp", given before init."""
        self.graph_path = path

    def init(self, workload: str, batch: int = 1, seed: int | None = None, seq_len: int = 0,
             dtype: str | None = None) -> None:
        if dtype is not None:
            self.dtype = dtype
        if workload in ("cc", "bfs", "pagerank", "sssp"):
            workload = workload + ":" + self.graph_path
        self.model = Model(workload, batch=batch, dtype=self.dtype, seq_len=seq_len)
        self.batch = batch
        if seed is not None:
            self.model.init_random(seed)
        check(B.load().gpx_exec_create(self.model.handle, self.KIND, ctypes.byref(self.handle)))

    def load_param(self, path: str) -> None:
        self.model.load_param(path)

    def set_input(self, key: str, value: np.ndarray, stream=None) -> None:
        self.model.set(key, value, stream)

    def get_output(self, key: str, stream=None) -> np.ndarray:
        return self.model.get(key, stream)

    def get_data_size(self, key: str) -> int:
        return self.model.get_storage_info(self.model.find_storage_idx(key))["size"]

    def get_kernel_num(self) -> int:
        return self.model.get_kernel_num()

    def execute(self, stream=None) -> None:
        check(B.load().gpx_exec_execute(self.handle, _h(stream)))

    def launch_kernel(self, kernel_offset: int, stream=None) -> None:
        check(B.load().gpx_exec_launch_kernel(self.handle, kernel_offset, _h(stream)))

    def capture_graph(self, stream) -> None:
        check(B.load().gpx_exec_capture_graph(self.handle, _h(stream)))

    def enable_trace(self, on: bool = True) -> None:
        check(B.load().gpx_exec_enable_trace(self.handle, int(on)))

    def read_trace(self) -> np.ndarray:
        n = ctypes.c_size_t()
        check(B.load().gpx_exec_read_trace(self.handle, None, 0, ctypes.byref(n)))
        out = np.empty(n.value, np.uint64)
        check(B.load().gpx_exec_read_trace(self.handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)),
                                           n.value, ctypes.byref(n)))
        return out.reshape(-1, 4)

    def error(self) -> tuple[int, int]:
        """(code, kernel*1000+cta) of a tensor-core kernel whose bounded wait gave up; (0, 0) = none."""
        code, where = ctypes.c_int(), ctypes.c_int()
        check(B.load().gpx_exec_error(self.handle, ctypes.byref(code), ctypes.byref(where)))
        return code.value, where.value

    def set_restart_policy(self, drop_tile_in_flight: bool) -> None:
        check(B.load().gpx_exec_set_restart_policy(self.handle, 1 if drop_tile_in_flight else 0))

    def reset_cursors(self, stream=None) -> None:
        check(B.load().gpx_exec_reset_cursors(self.handle, _h(stream)))

    def read_cursors(self) -> np.ndarray:
        n = ctypes.c_size_t()
        check(B.load().gpx_exec_read_cursors(self.handle, None, 0, ctypes.byref(n)))
        out = np.empty(n.value, np.int32)
        check(B.load().gpx_exec_read_cursors(self.handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int)),
                                             n.value, ctypes.byref(n)))
        return out

    def clear(self) -> None:
        if self.handle:
            B.load().gpx_exec_destroy(self.handle)
            self.handle = ctypes.c_void_p()
        if self.model is not None:
            self.model.clear()
            self.model = None


class BaseExecutor(Executor):
    """foo::BaseExecutor (include/executor.h:51-58)."""


class BLPExecutor(Executor):
    """foo::BLPExecutor (include/executor.h:60-84)."""

    KIND = B.EXEC_BLP

    def set_word(self, word: PreemptWord) -> None:
        """`blp_executor->dpStop = g_stop.d` (src/cuda-clients/blpclient.cpp:134)."""
        check(B.load().gpx_exec_set_word(self.handle, word.handle))

    def getStopPoint(self, stream=None) -> int:
        v = ctypes.c_int()
        check(B.load().gpx_exec_stop_point(self.handle, _h(stream), ctypes.byref(v)))
        return v.value

    def resume(self, stream=None) -> int:
        v = ctypes.c_int()
        check(B.load().gpx_exec_resume(self.handle, _h(stream), ctypes.byref(v)))
        return v.value


def run_workload(client: str, config_json: str) -> str:
    need = ctypes.c_size_t()
    cap = 1 << 20
    buf = ctypes.create_string_buffer(cap)
    st = B.load().gpx_run_workload(client.encode(), config_json.encode(), buf, cap, ctypes.byref(need))
    if st == B.OUT_OF_RANGE and need.value > cap:
        # the run completed; only the buffer was too small: fetch the kept report
        buf = ctypes.create_string_buffer(need.value)
        check(B.load().gpx_workload_report(buf, need.value, ctypes.byref(need)))
        return buf.value.decode()
    check(st)
    return buf.value.decode()


class _BorrowedStream:
    """A stream owned by the scheduler, usable wherever a Stream is (never destroyed here)."""

    def __init__(self, handle):
        self.handle = ctypes.c_void_p(handle)

    def sync(self) -> None:
        check(B.load().gpx_stream_sync(self.handle))


class Scheduler:
    """reef::executor::REEFScheduler (include/reef_scheduler.h:61-109): the per-GPU dispatch loop,
    for clients that bring their own request loop."""

    def __init__(self, device: int = 0, policy: str = "gpreemptclient"):
        self.handle = ctypes.c_void_p()
        check(B.load().gpx_sched_create(device, policy.encode(), ctypes.byref(self.handle)))

    def attach(self, executor: "Executor | None", priority: int) -> int:
        """create_queue + bind_model_queue: returns the client index."""
        c = ctypes.c_int()
        check(B.load().gpx_sched_attach(self.handle, executor.handle if executor is not None else None,
                                        priority, ctypes.byref(c)))
        return c.value

    def client_stream(self, client: int) -> _BorrowedStream:
        h = ctypes.c_void_p()
        check(B.load().gpx_sched_client_stream(self.handle, client, ctypes.byref(h)))
        return _BorrowedStream(h.value)

    def run(self) -> None:
        check(B.load().gpx_sched_run(self.handle))

    def shutdown(self) -> None:
        check(B.load().gpx_sched_shutdown(self.handle))

    def new_task(self, client: int) -> int:
        t = ctypes.c_uint64()
        check(B.load().gpx_sched_enqueue(self.handle, client, ctypes.byref(t)))
        return t.value

    def wait_task(self, client: int, ticket: int, timeout_s: float = 30.0) -> None:
        check(B.load().gpx_wait(self.handle, client, ticket, int(timeout_s * 1e9)))

    def hint(self, client: int, on: bool = True) -> None:
        check(B.load().gpx_sched_hint(self.handle, client, int(on)))

    def stats(self) -> dict:
        import json

        need = ctypes.c_size_t()
        check(B.load().gpx_sched_stats(self.handle, None, 0, ctypes.byref(need)))
        buf = ctypes.create_string_buffer(need.value)
        check(B.load().gpx_sched_stats(self.handle, buf, need.value, ctypes.byref(need)))
        return json.loads(buf.value.decode())

    def destroy(self) -> None:
        if self.handle:
            B.load().gpx_sched_destroy(self.handle)
            self.handle = ctypes.c_void_p()


def fill_uniform(buf: DeviceBuffer, n: int, bf16: bool, seed: int, stream_id: int = 0,
                 stream=None, lo: float = -1.0, hi: float = 1.0) -> None:
    """Fills a device buffer with the counter-based uniform generator (fp32 or bf16)."""
    check(B.load().gpx_fill_uniform(buf.ptr, n, int(bf16), seed, stream_id, lo, hi, _h(stream)))
    check(B.load().gpx_stream_sync(_h(stream)))


def count_diff(a: DeviceBuffer, b: DeviceBuffer, nbytes: int, stream=None) -> int:
    d = ctypes.c_uint64()
    check(B.load().gpx_count_diff(a.ptr, b.ptr, nbytes, ctypes.byref(d), _h(stream)))
    return d.value


def preempt_microbench(kind: str, size: int, triggers: int, seed: int = 5,
                       transport: int = B.WORD_DEVICE) -> dict:
    """Runs gpx_preempt_microbench; kind is "axpy" (size = elements) or "gemm" (size = M=N=K)."""
    summary = B.MicrobenchSummary()
    drain = (ctypes.c_double * max(triggers, 1))()
    seen = (ctypes.c_double * max(triggers, 1))()
    check(B.load().gpx_preempt_microbench(0 if kind == "axpy" else 1, size, triggers, seed,
                                          transport, drain, seen, ctypes.byref(summary)))
    out = {name: getattr(summary, name) for name, _ in B.MicrobenchSummary._fields_}
    out["drain_us"] = list(drain[:summary.preempted])
    out["seen_us"] = list(seen[:summary.preempted])
    return out


def clock_offset_ns() -> tuple[int, int]:
    off, unc = ctypes.c_int64(), ctypes.c_int64()
    check(B.load().gpx_clock_offset_ns(ctypes.byref(off), ctypes.byref(unc)))
    return off.value, unc.value


def host_now_ns() -> int:
    return B.load().gpx_host_now_ns()
