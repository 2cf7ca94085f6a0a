"""ctypes declarations of every entry point in include/gpx.h."""
from __future__ import annotations

import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
# GPX_LIB selects another build of the library (a development variant made with
# `python -m gpreempt_b200.build --define ... --out DIR`).
LIB_PATH = os.environ.get("GPX_LIB") or os.path.join(HERE, "lib", "libgpx.so")
HEADER = os.path.join(HERE, "..", "include", "gpx.h")

SUCC, FAIL, TIMEOUT, NOT_FOUND, OUT_OF_RANGE, FULL = range(6)
WORD_MAPPED, WORD_DEVICE = 0, 1
EXEC_BASE, EXEC_BLP = 0, 1


class GpxError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"gpx status {status}: {text}")
        self.status = status


class Blp(ctypes.Structure):
    _fields_ = [
        ("preempted", ctypes.c_void_p),
        ("stop_index", ctypes.c_void_p),
        ("executed", ctypes.c_void_p),
        ("kernel_id", ctypes.c_int),
        ("trace", ctypes.c_void_p),
    ]


class MicrobenchSummary(ctypes.Structure):
    _fields_ = [
        ("triggers", ctypes.c_int), ("preempted", ctypes.c_int), ("resumes", ctypes.c_int),
        ("mismatches", ctypes.c_int), ("kernel_ms", ctypes.c_double),
        ("drain_us_p50", ctypes.c_double), ("drain_us_p99", ctypes.c_double),
        ("drain_us_max", ctypes.c_double), ("drain_us_mean", ctypes.c_double),
        ("seen_us_p50", ctypes.c_double), ("seen_us_p99", ctypes.c_double),
        ("clock_uncertainty_ns", ctypes.c_double),
        ("raise_call_us_p50", ctypes.c_double), ("raise_call_us_max", ctypes.c_double),
        ("drain_after_return_us_max", ctypes.c_double), ("late_starts", ctypes.c_int),
    ]


class ModelOpts(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int), ("dtype", ctypes.c_char_p), ("seq_len", ctypes.c_int)]


def declared_symbols() -> list[str]:
    """Names of all functions include/gpx.h declares."""
    with open(HEADER) as fp:
        text = fp.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gpx_[a-z0-9_]+)\s*\(", text)))


_lib = None

vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
u64, i64 = ctypes.c_uint64, ctypes.c_int64
P = ctypes.POINTER

_SIGS = {
    "gpx_init": [ci],
    "gpx_device_count": [P(ci)],
    "gpx_device_info": [P(ci), P(sz), ctypes.c_char_p, sz],
    "gpx_bind_core": [ci],
    "gpx_malloc": [P(vp), sz],
    "gpx_free": [vp],
    "gpx_host_alloc": [P(vp), sz],
    "gpx_host_free": [vp],
    "gpx_memcpy_h2d": [vp, vp, sz, vp],
    "gpx_memcpy_d2h": [vp, vp, sz, vp],
    "gpx_memcpy_d2d": [vp, vp, sz, vp],
    "gpx_memset": [vp, ci, sz, vp],
    "gpx_stream_create": [P(vp), ci],
    "gpx_stream_destroy": [vp],
    "gpx_stream_sync": [vp],
    "gpx_stream_query": [vp],
    "gpx_device_sync": [],
    "gpx_event_create": [P(vp)],
    "gpx_event_destroy": [vp],
    "gpx_event_record": [vp, vp],
    "gpx_event_sync": [vp],
    "gpx_event_elapsed_ms": [vp, vp, P(ctypes.c_float)],
    "gpx_set_priority": [ci],
    "gpx_word_create": [P(vp), ci],
    "gpx_word_destroy": [vp],
    "gpx_word_raise": [vp],
    "gpx_word_clear": [vp],
    "gpx_word_dptr": [vp, P(vp)],
    "gpx_word_value": [vp, P(ci)],
    "gpx_block_launch": [vp, vp, u64, vp],
    "gpx_noop_launch": [vp],
    "gpx_axpy_f32": [ctypes.c_float, vp, vp, sz, sz, P(Blp), vp],
    "gpx_axpy_tiles": [sz, sz, P(ci)],
    "gpx_gemm_bf16": [vp, vp, vp, ci, ci, ci, vp, P(Blp), vp],
    "gpx_gemm_ctx_bytes": [P(sz)],
    "gpx_gemm_tiles": [ci, ci, P(ci)],
    "gpx_gemm_status": [vp, P(ci), P(ci)],
    "gpx_gemm_bf16_static": [vp, vp, vp, ci, ci, ci, ci, P(Blp), vp],
    "gpx_gemm_static_status": [P(ci), P(ci)],
    "gpx_preempt_microbench": [ci, sz, ci, u64, ci, P(ctypes.c_double), P(ctypes.c_double),
                               P(MicrobenchSummary)],
    "gpx_fill_uniform": [vp, sz, ci, u64, u64, ctypes.c_float, ctypes.c_float, vp],
    "gpx_count_diff": [vp, vp, sz, P(u64), vp],
    "gpx_synth_normal": [vp, sz, u64, u64, ctypes.c_float, ctypes.c_float],
    "gpx_synth_uniform": [vp, sz, u64, u64, ctypes.c_float, ctypes.c_float],
    "gpx_model_open": [ctypes.c_char_p, P(ModelOpts), P(vp)],
    "gpx_model_close": [vp],
    "gpx_model_load_params": [vp, ctypes.c_char_p],
    "gpx_model_save_params": [vp, ctypes.c_char_p],
    "gpx_model_init_random": [vp, u64],
    "gpx_model_storage_num": [vp, P(sz)],
    "gpx_model_storage_info": [vp, sz, ctypes.c_char_p, sz, P(sz), ctypes.c_char_p, sz, P(ci)],
    "gpx_model_find": [vp, ctypes.c_char_p, P(sz)],
    "gpx_model_set": [vp, ctypes.c_char_p, vp, sz, vp],
    "gpx_model_get": [vp, ctypes.c_char_p, vp, sz, vp],
    "gpx_model_shape": [vp, ctypes.c_char_p, P(i64), P(ci)],
    "gpx_model_kernel_num": [vp, P(sz)],
    "gpx_model_kernel_info": [vp, sz, ctypes.c_char_p, sz, P(ctypes.c_uint32), P(ci),
                              P(ctypes.c_double), P(ctypes.c_double)],
    "gpx_model_export_json": [vp, ctypes.c_char_p, sz, P(sz)],
    "gpx_model_export_dir": [vp, ctypes.c_char_p],
    "gpx_model_reductions": [vp, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)],
    "gpx_model_graph_info": [vp, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64),
                             ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)],
    "gpx_exec_create": [vp, ci, P(vp)],
    "gpx_exec_destroy": [vp],
    "gpx_exec_set_word": [vp, vp],
    "gpx_exec_set_word_dptr": [vp, vp],
    "gpx_exec_execute": [vp, vp],
    "gpx_exec_launch_kernel": [vp, sz, vp],
    "gpx_exec_capture_graph": [vp, vp],
    "gpx_exec_stop_point": [vp, vp, P(ci)],
    "gpx_exec_resume": [vp, vp, P(ci)],
    "gpx_exec_enable_trace": [vp, ci],
    "gpx_exec_read_trace": [vp, P(u64), sz, P(sz)],
    "gpx_launch_count": [P(u64)],
    "gpx_exec_cursor_dptr": [vp, P(vp)],
    "gpx_exec_error": [vp, P(ci), P(ci)],
    "gpx_exec_reset_cursors": [vp, vp],
    "gpx_exec_set_restart_policy": [vp, ctypes.c_int],
    "gpx_exec_read_cursors": [vp, P(ci), sz, P(sz)],
    "gpx_run_workload": [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p, sz, P(sz)],
    "gpx_workload_report": [ctypes.c_char_p, sz, P(sz)],
    "gpx_sched_create": [ci, ctypes.c_char_p, P(vp)],
    "gpx_sched_attach": [vp, vp, ci, P(ci)],
    "gpx_sched_client_stream": [vp, ci, P(vp)],
    "gpx_sched_run": [vp],
    "gpx_sched_shutdown": [vp],
    "gpx_sched_destroy": [vp],
    "gpx_sched_enqueue": [vp, ci, P(u64)],
    "gpx_wait": [vp, ci, u64, u64],
    "gpx_sched_hint": [vp, ci, ci],
    "gpx_sched_stats": [vp, ctypes.c_char_p, sz, P(sz)],
    "gpx_clock_offset_ns": [P(i64), P(i64)],
}


def load() -> ctypes.CDLL:
    """Loads libgpx.so; raises when it has not been built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m gpreempt_b200.build`; "
            "gpreempt_b200 has no CPU or PyTorch fallback")
    lib = ctypes.CDLL(LIB_PATH)
    for name, args in _SIGS.items():
        if not hasattr(lib, name):
            continue
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ci
    lib.gpx_strerror.argtypes = [ci]
    lib.gpx_strerror.restype = ctypes.c_char_p
    lib.gpx_last_error.argtypes = []
    lib.gpx_last_error.restype = ctypes.c_char_p
    lib.gpx_host_now_ns.argtypes = []
    lib.gpx_host_now_ns.restype = u64
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != SUCC:
        lib = load()
        text = lib.gpx_last_error().decode(errors="replace")
        raise GpxError(status, f"{lib.gpx_strerror(status).decode()}: {text}")
