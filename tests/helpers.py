"""Shared comparison logic for the parity tests."""
from __future__ import annotations

import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def sorted_pairs(pairs):
    a = np.asarray(pairs, dtype=np.uint32).reshape(-1, 2)
    return a[np.lexsort((a[:, 1], a[:, 0]))]


def run_and_collect(runner, net, steps, dump_every, step_fn=None):
    """Step `runner` (oracle or CUDA runtime: both expose step/array/
    current_spikes) and collect what the golden fixtures hold, under the same
    keys the reference driver uses."""
    out = {}
    spikes = {p.name: [] for p in net.pops}
    step = step_fn or (lambda n: runner.step(n))
    for s in range(steps):
        step(1)
        for p in net.pops:
            ids = runner.current_spikes(p.name)
            spikes[p.name] += [(s, int(i)) for i in ids]
        if (s + 1) % dump_every == 0:
            out.update(snapshot(runner, net, s + 1))
    for name, sp in spikes.items():
        out[f"spikes_{name}"] = sorted_pairs(sp)
    return out


def snapshot(runner, net, step):
    out = {}
    for p in net.pops:
        if p.kind == "LIF":
            out[f"V_{p.name}_{step}"] = runner.array(f"{p.name}.V")[0]
            out[f"RefracTime_{p.name}_{step}"] = runner.array(f"{p.name}.RefracTime")[0]
        elif p.kind == "Izhikevich":
            out[f"V_{p.name}_{step}"] = runner.array(f"{p.name}.V")[0]
            out[f"U_{p.name}_{step}"] = runner.array(f"{p.name}.U")[0]
    for i, psm in enumerate(net.psms):
        # the reference keeps a fused buffer under the name of the last group fused into it
        out[f"outPost_{psm.members[-1]}_{step}"] = runner.array(f"psm{i}.out_post")[0]
    for s in net.syns:
        if s.wum == "STDP":
            out[f"g_{s.name}_{step}"] = runner.array(f"{s.name}.g")[0]
    return out


def input_scale(net, name):
    """Sum of |weight| that can reach one postsynaptic buffer: the scale the
    1e-5 tolerance on summed input is relative to (contributions of opposite
    sign cancel, so the error is relative to what was added, not to what is left)."""
    return 1.0


def assert_close(got, want, key, rtol, atol):
    assert got.shape == want.shape, f"{key}: shape {got.shape} vs {want.shape}"
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bound = atol + rtol * np.abs(want.astype(np.float64))
    bad = np.nonzero(err > bound)[0]
    assert len(bad) == 0, (f"{key}: {len(bad)} of {len(want)} elements differ, worst |err|={err.max():.3e} "
                           f"at {int(err.argmax())} (got {got[err.argmax()]}, want {want[err.argmax()]})")


def compare(got, want, exact_state, rtol=1e-5, atol=1e-6):
    """Spike (step, id) sets always bit-exact; state exact or within tolerance."""
    for key, w in want.items():
        assert key in got, f"missing {key}"
        g = got[key]
        if key.startswith("spikes_"):
            assert g.shape == w.shape and np.array_equal(g, w), \
                f"{key}: spike sets differ ({len(g)} vs {len(w)} spikes)"
        elif exact_state:
            assert np.array_equal(g, w), f"{key}: not bit-identical (max |err| {np.abs(g - w).max():.3e})"
        else:
            assert_close(g, w, key, rtol, atol)
