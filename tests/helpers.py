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


class ContributionScale:
    """Per postsynaptic buffer and target neuron, the running sum of |weight| of everything that was
    added into the buffer, decayed as the buffer itself decays: the magnitude the 1e-5 tolerance on
    a summed input is relative to.  Contributions of opposite sign cancel, so the rounding error of
    an unordered fp32 sum scales with what was added, not with what is left of it.

    Call :meth:`step` once per simulated step with the spikes emitted in the step BEFORE it (the ones
    that step's synapse update propagates), in the order of the simulator: synapses into buffer or
    ring slot, then the neuron update consumes the front slot and decays the buffer."""

    def __init__(self, net):
        self.net = net
        self.k = 0
        self.history = []           # spikes by population, newest last
        self.acc = [np.zeros(net.pop(p.trg).n) for p in net.psms]
        self.ring = [np.zeros((p.max_den_delay, net.pop(p.trg).n)) if p.max_den_delay else None for p in net.psms]
        self.decay = [float(p.derived.get("expDecay", 0.0)) for p in net.psms]

    def step(self, spikes_by_pop):
        net = self.net
        self.history.append({k: np.asarray(v, dtype=np.int64) for k, v in spikes_by_pop.items()})
        for s in net.syns:
            if s.matrix != "SPARSE" or s.ind is None or len(self.history) <= s.ax_delay:
                continue
            psm = net.psms[s.psm]
            for pre in self.history[-1 - s.ax_delay].get(s.src, ()):
                lo = int(pre) * s.row_stride
                n = int(s.row_length[pre])
                post = np.asarray(s.ind[lo:lo + n], dtype=np.int64)
                w = (np.abs(np.asarray(s.g[lo:lo + n], dtype=np.float64)) if s.g is not None
                     else np.full(n, abs(float(s.wum_params["g"]))))
                if s.max_den_delay:
                    D = psm.max_den_delay
                    slot = (self.k + 1 + np.asarray(s.d[lo:lo + n], dtype=np.int64)) % D
                    np.add.at(self.ring[s.psm], (slot, post), w)
                else:
                    np.add.at(self.acc[s.psm], post, w)
        self.k += 1
        for i, psm in enumerate(net.psms):
            if self.ring[i] is not None:
                front = self.k % psm.max_den_delay
                self.acc[i] += self.ring[i][front]
                self.ring[i][front] = 0.0
            self.acc[i] *= self.decay[i]

    def scale(self, psm_index):
        return self.acc[psm_index]


def assert_close(got, want, key, rtol, atol, scale=None):
    """|got - want| <= atol + rtol * max(|want|, scale): `scale` (per element) widens the relative
    bound to the magnitude of what was summed into the element."""
    assert got.shape == want.shape, f"{key}: shape {got.shape} vs {want.shape}"
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    ref = np.abs(want.astype(np.float64))
    if scale is not None:
        ref = np.maximum(ref, np.broadcast_to(scale, ref.shape))
    bound = atol + rtol * ref
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
