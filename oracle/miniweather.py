"""ctypes wrapper of the miniWeather CPU oracle (miniweather_oracle.c) - TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and bench.py's CPU baseline may import this module.  `Reference`
wraps oracle/_ref/libminiweather_ref.so, the reference's own CUDA source compiled unmodified
(oracle/Makefile, target `ref`); it needs a GPU and exists only where that library was built.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libminiweather_oracle.so")
REF_LIB_PATH = os.path.join(_HERE, "_ref", "libminiweather_ref.so")
_lib = None
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)

HALO = 2
NUM_VARS = 4
ID_DENS, ID_UMOM, ID_WMOM, ID_RHOT = range(4)


def build() -> str:
    src = os.path.join(_HERE, "miniweather_oracle.c")
    if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libminiweather_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.mwo_create.restype = ctypes.c_void_p
        _lib.mwo_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
        _lib.mwo_destroy.argtypes = [ctypes.c_void_p]
        _lib.mwo_timestep.argtypes = [ctypes.c_void_p]
        _lib.mwo_timestep_upto.argtypes = [ctypes.c_void_p, ctypes.c_int]
        for name in ("mwo_state", "mwo_state_tmp"):
            getattr(_lib, name).restype = _f32p
            getattr(_lib, name).argtypes = [ctypes.c_void_p]
        _lib.mwo_field.restype = _f32p
        _lib.mwo_field.argtypes = [ctypes.c_void_p, ctypes.c_int]
        _lib.mwo_dt.restype = ctypes.c_float
        _lib.mwo_dt.argtypes = [ctypes.c_void_p]
        _lib.mwo_reductions.argtypes = [ctypes.c_void_p, _f64p, _f64p]
    return _lib


class Oracle:
    """The reference's simulation on the CPU: `state` is a view [4][nz+4][nx+4] of the live array."""

    FIELDS = {"hy_dens_cell": 0, "hy_dens_theta_cell": 1, "hy_dens_int": 2, "hy_dens_theta_int": 3,
              "hy_pressure_int": 4, "hy_dens_cell_const": 5}

    def __init__(self, nx: int, nz: int, full_halo: bool = False):
        self.nx, self.nz = nx, nz
        self._h = lib().mwo_create(nx, nz, 1 if full_halo else 0)
        self.shape = (NUM_VARS, nz + 2 * HALO, nx + 2 * HALO)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().mwo_destroy(self._h)
            self._h = None

    def _view(self, ptr) -> np.ndarray:
        return np.ctypeslib.as_array(ptr, shape=self.shape)

    @property
    def state(self) -> np.ndarray:
        return self._view(lib().mwo_state(self._h))

    @property
    def state_tmp(self) -> np.ndarray:
        return self._view(lib().mwo_state_tmp(self._h))

    @property
    def dt(self) -> float:
        return float(lib().mwo_dt(self._h))

    def field(self, name: str) -> np.ndarray:
        n = {"hy_dens_cell": self.nz + 4, "hy_dens_theta_cell": self.nz + 4, "hy_dens_cell_const": 4}.get(name, self.nz + 1)
        return np.ctypeslib.as_array(lib().mwo_field(self._h, self.FIELDS[name]), shape=(n,))

    def timestep(self, n: int = 1) -> None:
        for _ in range(n):
            lib().mwo_timestep(self._h)

    def timestep_upto(self, semi_steps: int) -> None:
        lib().mwo_timestep_upto(self._h, semi_steps)

    def reductions(self) -> tuple[float, float]:
        mass, te = ctypes.c_double(), ctypes.c_double()
        lib().mwo_reductions(self._h, ctypes.byref(mass), ctypes.byref(te))
        return mass.value, te.value


def interior(state: np.ndarray) -> np.ndarray:
    return state[:, HALO:-HALO, HALO:-HALO]


def reference_available() -> bool:
    return os.path.exists(REF_LIB_PATH)


class Reference:
    """The reference's own kernels (3200 x 1600 cells) on the current GPU."""

    def __init__(self, device: int = 0):
        self._lib = ctypes.CDLL(REF_LIB_PATH)
        self._lib.mwref_state.argtypes = [ctypes.c_int, _f32p, ctypes.c_size_t]
        self._lib.mwref_dt.restype = ctypes.c_float
        self._lib.mwref_time_steps.restype = ctypes.c_float
        self._lib.mwref_time_steps.argtypes = [ctypes.c_int]
        self._lib.mwref_reductions.argtypes = [_f64p, _f64p]
        nx, nz = ctypes.c_int(), ctypes.c_int()
        self._lib.mwref_grid(ctypes.byref(nx), ctypes.byref(nz))
        self.nx, self.nz = nx.value, nz.value
        self.shape = (NUM_VARS, self.nz + 2 * HALO, self.nx + 2 * HALO)
        if self._lib.mwref_init(device) != 0:
            raise RuntimeError("reference miniWeather failed to initialise")

    def timestep(self, n: int = 1) -> None:
        if self._lib.mwref_steps(n) != 0:
            raise RuntimeError("reference miniWeather step failed")

    def time_steps(self, n: int) -> float:
        """Device milliseconds of n time steps (they advance the state)."""
        ms = float(self._lib.mwref_time_steps(n))
        if ms < 0:
            raise RuntimeError("reference miniWeather timing failed")
        return ms

    def state(self, which: int = 0) -> np.ndarray:
        out = np.empty(self.shape, dtype=np.float32)
        if self._lib.mwref_state(which, out.ctypes.data_as(_f32p), out.size) != 0:
            raise RuntimeError("reference miniWeather state read failed")
        return out

    @property
    def dt(self) -> float:
        return float(self._lib.mwref_dt())

    def reductions(self) -> tuple[float, float]:
        mass, te = ctypes.c_double(), ctypes.c_double()
        if self._lib.mwref_reductions(ctypes.byref(mass), ctypes.byref(te)) != 0:
            raise RuntimeError("reference miniWeather reductions failed")
        return mass.value, te.value

    def close(self) -> None:
        self._lib.mwref_finalize()
