"""Writes tests/golden/miniweather_reference.json from the reference's own miniWeather kernels.

Run where a GPU is, after `make -C oracle ref` built oracle/_ref/libminiweather_ref.so from the
reference's unmodified src/workloads/miniweather.cu:

    python tests/golden/make_miniweather_golden.py

For 0, 1 and 3 time steps on the reference's 3200 x 1600 grid the file keeps the domain mass and
total energy (reductions), per-variable sums and extrema of the interior, and the four variables
at 48 fixed cells, so the CPU oracle can be checked where no GPU is.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import miniweather as mw  # noqa: E402

OUT = os.path.join(ROOT, "tests", "golden", "miniweather_reference.json")


def sample_cells(nx, nz):
    rng = np.random.default_rng(20240607)
    ks = rng.integers(0, nz, 40).tolist() + [0, 1, nz - 2, nz - 1, 0, nz - 1, 800, 800]
    is_ = rng.integers(0, nx, 40).tolist() + [5, nx - 1, 0, 77, 1600, 1599, 0, nx - 1]
    return list(zip(ks, is_))


def summary(state, cells):
    inner = mw.interior(state).astype(np.float64)
    return {
        "sum": [float(inner[v].sum()) for v in range(4)],
        "abs_sum": [float(np.abs(inner[v]).sum()) for v in range(4)],
        "min": [float(inner[v].min()) for v in range(4)],
        "max": [float(inner[v].max()) for v in range(4)],
        "cells": [[float(state[v, k + 2, i + 2]) for v in range(4)] for k, i in cells],
        "halo_rows": {"dens_row0": float(state[0, 0, 1000]), "umom_row0_col50": float(state[1, 0, 50]),
                      "umom_row0_col2000": float(state[1, 0, 2000]), "rhot_row0": float(state[3, 0, 1000]),
                      "rhot_top": float(state[3, -1, 1000])},
    }


def main():
    ref = mw.Reference(0)
    cells = sample_cells(ref.nx, ref.nz)
    doc = {"source": "reference src/workloads/miniweather.cu compiled unmodified (oracle/Makefile, target ref)",
           "nx": ref.nx, "nz": ref.nz, "dt": ref.dt, "cells": cells, "steps": {}}
    done = 0
    for steps in (0, 1, 3):
        ref.timestep(steps - done)
        done = steps
        mass, te = ref.reductions()
        s = summary(ref.state(0), cells)
        s["mass"], s["te"] = mass, te
        doc["steps"][str(steps)] = s
    ref.timestep(2)  # warm
    doc["reference_ms_per_time_step_on_this_gpu"] = ref.time_steps(20) / 20
    print("reference: %.3f ms per time step" % doc["reference_ms_per_time_step_on_this_gpu"])
    ref.close()
    with open(OUT, "w") as fp:
        json.dump(doc, fp, indent=1)
    print("wrote", OUT)


if __name__ == "__main__":
    main()
