"""Network descriptions for the plug-in tests: text specs (the format oracle/ref_driver.cc reads)
of small networks driven through the UNMODIFIED GeNN front end and runtime, once with GeNN's own
single_threaded_cpu backend and once with the B200 code-generation backend.

`custom_models` uses a neuron model and a weight update model that are NOT built into GeNN
(their code strings are defined in the driver), so nothing but the transpiled strings can have
produced the kernels' arithmetic."""
from __future__ import annotations

import os

import numpy as np

from genn_b200 import workloads


def _dump(directory, name, arr):
    np.ascontiguousarray(arr).tofile(os.path.join(directory, name))
    return name


def _ragged(rng, num_pre, num_post, prob):
    mask = rng.random((num_pre, num_post)) < prob
    row_length = mask.sum(axis=1).astype(np.uint32)
    stride = int(max(1, row_length.max()))
    ind = np.zeros((num_pre, stride), dtype=np.uint32)
    for i in range(num_pre):
        ind[i, :row_length[i]] = np.nonzero(mask[i])[0]
    return row_length, stride, ind, mask


def custom_models(directory: str, steps: int = 400, dump_every: int = 100) -> str:
    """Spike sources -> 300 adaptive quadratic integrate-and-fire neurons through SPARSE connectivity
    with a scaled, saturating pulse rule; the population also excites itself through a second group
    of the same rule (recurrent, so errors would compound)."""
    os.makedirs(directory, exist_ok=True)
    rng = np.random.default_rng(42)
    n_in, n = 120, 300
    start, end, times = workloads.poisson_spike_trains(rng, n_in, 60.0, steps * 0.5)
    lines = ["name custom_models", "dt 0.5", "seed 1234", f"steps {steps}", f"dump_every {dump_every}",
             "fuse_psm 0", "narrow_ind 0"]
    lines.append(f"pop in {n_in} SSA " + _dump(directory, "start_in.bin", start) + " " + _dump(directory, "end_in.bin", end)
                 + " " + _dump(directory, "times_in.bin", times))
    # C, k, Vrest, Vcrit, Vpeak, Vreset, a, b, tauW, Ioffset
    params = "100.0 0.7 -60.0 -40.0 35.0 -50.0 0.03 20.0 100.0 40.0"
    v0 = rng.uniform(-65.0, -55.0, n).astype(np.float32)
    w0 = np.zeros(n, dtype=np.float32)
    lines.append(f"pop q {n} AQIF {params} " + _dump(directory, "V_q.bin", v0) + " " + _dump(directory, "W_q.bin", w0))
    rl, stride, ind, mask = _ragged(rng, n_in, n, 0.15)
    g = np.zeros((n_in, stride), dtype=np.float32)
    g[np.arange(stride)[None, :] < rl[:, None]] = rng.uniform(20.0, 120.0, int(rl.sum())).astype(np.float32)
    lines.append(f"syn ff SPARSE in q wum SCALED 1.5 150.0 psm EXPCURR 4.0 maxconn {stride} rowlength "
                 + _dump(directory, "rl_ff.bin", rl) + " ind " + _dump(directory, "ind_ff.bin", ind) + " g " + _dump(directory, "g_ff.bin", g))
    rl2, stride2, ind2, _ = _ragged(rng, n, n, 0.05)
    g2 = np.zeros((n, stride2), dtype=np.float32)
    g2[np.arange(stride2)[None, :] < rl2[:, None]] = rng.uniform(5.0, 40.0, int(rl2.sum())).astype(np.float32)
    lines.append(f"syn rec SPARSE q q wum SCALED 0.8 25.0 psm EXPCURR 6.0 maxconn {stride2} rowlength "
                 + _dump(directory, "rl_rec.bin", rl2) + " ind " + _dump(directory, "ind_rec.bin", ind2) + " g " + _dump(directory, "g_rec.bin", g2))
    path = os.path.join(directory, "spec.txt")
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    return path
