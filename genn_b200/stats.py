"""Spike-train statistics of a recorded run: per-population mean firing rate
and mean coefficient of variation of the inter-spike intervals.

These are the quantities recurrent (chaotic) networks are compared on: two
correct simulators diverge spike by spike after a few hundred steps, but the
population statistics of the asynchronous state agree.
"""
from __future__ import annotations

from typing import Dict

import numpy as np


def partial(steps: np.ndarray, ids: np.ndarray, num_neurons: int, first_id: int = 0, min_spikes: int = 3):
    """Sums from which rate and CV-ISI of a population follow, for one slice of its neurons
    (ids ``first_id .. first_id + num_neurons``): [spikes, neurons, sum of per-neuron CVs, neurons in
    that sum].  Slices held by different processes add up element by element."""
    steps = np.asarray(steps, dtype=np.int64)
    ids = np.asarray(ids, dtype=np.int64) - first_id
    order = np.lexsort((steps, ids))
    s, i = steps[order], ids[order]
    same = i[1:] == i[:-1]
    isi = (s[1:] - s[:-1])[same].astype(np.float64)
    owner = i[1:][same]
    n_isi = np.bincount(owner, minlength=num_neurons).astype(np.float64)
    sum1 = np.bincount(owner, weights=isi, minlength=num_neurons)
    sum2 = np.bincount(owner, weights=isi * isi, minlength=num_neurons)
    ok = n_isi >= (min_spikes - 1)
    mean = sum1[ok] / n_isi[ok]
    var = np.maximum(sum2[ok] / n_isi[ok] - mean * mean, 0.0)
    cv = np.sqrt(var) / mean
    return np.array([float(len(ids)), float(num_neurons), float(cv.sum()), float(ok.sum())])


def merge(partials, duration_s: float) -> Dict[str, float]:
    t = np.sum(np.asarray(partials, dtype=np.float64).reshape(-1, 4), axis=0)
    return {"rate_hz": float(t[0] / max(1.0, t[1]) / duration_s),
            "cv_isi": float(t[2] / t[3]) if t[3] > 0 else float("nan"),
            "neurons_in_cv": int(t[3]), "spikes": int(t[0])}


def rate_and_cv(steps: np.ndarray, ids: np.ndarray, num_neurons: int, duration_s: float,
                first_id: int = 0, min_spikes: int = 3) -> Dict[str, float]:
    """``steps``/``ids``: one entry per spike (time step, neuron id).  Rate is
    spikes / neuron / second over all ``num_neurons``; CV-ISI is the mean over
    the neurons with at least ``min_spikes`` spikes of std(ISI) / mean(ISI)
    (population standard deviation, intervals in time steps)."""
    return merge([partial(steps, ids, num_neurons, first_id, min_spikes)], duration_s)


def compare(got: Dict[str, Dict[str, float]], want: Dict[str, Dict[str, float]]):
    """Largest relative error of rate and of CV-ISI over the populations."""
    r = max(abs(got[p]["rate_hz"] - want[p]["rate_hz"]) / want[p]["rate_hz"] for p in want)
    c = max(abs(got[p]["cv_isi"] - want[p]["cv_isi"]) / want[p]["cv_isi"] for p in want)
    return float(r), float(c)
