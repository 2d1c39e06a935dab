"""Small seeded networks used by the golden-vector generator, the CPU-checker
tests and the GPU parity tests.  Each builder returns (GeNNModel, steps,
dump_every); all of them are free of random draws inside the simulation so the
reference's CPU backend, the C checker and the CUDA kernels see identical
inputs."""
from __future__ import annotations

import numpy as np

from genn_b200 import GeNNModel, init_postsynaptic, init_weight_update, workloads


def ff_sparse():
    return workloads.feedforward(seed=3, num_pre=200, num_post=500, prob=0.1, rate_hz=200.0, steps=300), 300, 50


def c1_full():
    """Benchmark config 1 at its stated size: 1 000 spike sources at 20 Hz (host-generated trains)
    -> 10 000 LIF through SPARSE p = 0.1 (about 1 M synapses), weights U[0, 0.05) nA, exponential
    current synapses with tau 5 ms, 1 000 steps of 0.1 ms."""
    return workloads.feedforward(seed=1, num_pre=1000, num_post=10000, prob=0.1, rate_hz=20.0, steps=1000), 1000, 250


def ff_sparse_narrow():
    m = workloads.feedforward(seed=4, num_pre=150, num_post=200, prob=0.2, rate_hz=200.0, steps=300, narrow=True)
    return m, 300, 50


def ff_bitmask():
    return workloads.feedforward(seed=5, num_pre=200, num_post=333, prob=0.1, rate_hz=200.0, steps=300,
                                 matrix="BITMASK"), 300, 50


def ff_dense():
    return workloads.feedforward(seed=6, num_pre=64, num_post=300, prob=0.3, rate_hz=200.0, steps=300,
                                 matrix="DENSE"), 300, 50


def potjans_mini():
    """Potjans architecture at 0.5% of the neurons, constant-current background
    (no random draws in the loop), host-drawn connectivity, weights, delays."""
    m = workloads.potjans(neuron_scale=0.005, seed=7, host_connectivity=True, background="dc", record=True)
    return m, 400, 100


def potjans_mini_d1():
    """The same with every delay at least one step (lower clip dt instead of 0) and
    a ring one slot longer than the longest delay, so that no synapse wraps around
    it: the persistent kernel may then deliver spikes one step late."""
    m = workloads.potjans(neuron_scale=0.005, seed=7, host_connectivity=True, background="dc", record=True,
                          min_delay=0.1, extra_delay_slots=1)
    return m, 400, 100


def cond_delay():
    """Recurrent conductance-based E/I network with a 1 ms axonal delay and
    constant weights (config 2 in miniature)."""
    rng = np.random.default_rng(8)
    m = GeNNModel("float", "cond_delay")
    m.dt = 0.1
    lif = {"C": 0.2, "TauM": 20.0, "Vrest": -60.0, "Vreset": -60.0, "Vthresh": -50.0, "Ioffset": 0.25,
           "TauRefrac": 5.0}
    ne, ni, k = 400, 100, 40
    e = m.add_neuron_population("E", ne, "LIF", lif, {"V": rng.uniform(-60, -50, ne).astype(np.float32), "RefracTime": 0.0})
    i = m.add_neuron_population("I", ni, "LIF", lif, {"V": rng.uniform(-60, -50, ni).astype(np.float32), "RefracTime": 0.0})
    e.spike_recording_enabled = True
    i.spike_recording_enabled = True
    for src, w, tau, erev in ((e, 0.0006 * 10, 5.0, 0.0), (i, 0.0067 * 10, 10.0, -80.0)):
        for trg in (e, i):
            post = np.repeat(np.arange(trg.num_neurons, dtype=np.uint32), k)
            pre = rng.integers(0, src.num_neurons, size=len(post)).astype(np.uint32)
            sg = m.add_synapse_population(f"{src.name}{trg.name}", "SPARSE", src, trg,
                                          init_weight_update("StaticPulseConstantWeight", {"g": w}),
                                          init_postsynaptic("ExpCond", {"tau": tau, "E": erev}))
            sg.set_sparse_connections(pre, post)
            sg.axonal_delay_steps = 10
    return m, 400, 100


def stdp():
    """Spike sources -> LIF through SPARSE connectivity with additive STDP."""
    rng = np.random.default_rng(9)
    m = GeNNModel("float", "stdp")
    m.dt = 1.0
    npre, npost, steps = 120, 60, 300
    start, end, times = workloads.poisson_spike_trains(rng, npre, 40.0, steps * m.dt)
    src = m.add_neuron_population("pre", npre, "SpikeSourceArray", {}, {"startSpike": start, "endSpike": end})
    src.set_extra_global_param("spikeTimes", times)
    lif = {"C": 1.0, "TauM": 20.0, "Vrest": -65.0, "Vreset": -70.0, "Vthresh": -55.0, "Ioffset": 0.0, "TauRefrac": 2.0}
    trg = m.add_neuron_population("post", npost, "LIF", lif, {"V": -65.0, "RefracTime": 0.0})
    src.spike_recording_enabled = True
    trg.spike_recording_enabled = True
    mask = rng.random((npre, npost)) < 0.4
    pre, post = np.nonzero(mask)
    g = rng.uniform(0.0, 0.5, size=len(pre)).astype(np.float32)
    sg = m.add_synapse_population("syn", "SPARSE", src, trg,
                                  init_weight_update("STDP", {"tauPlus": 20.0, "tauMinus": 20.0, "Aplus": 0.01,
                                                              "Aminus": 0.0105, "Wmin": 0.0, "Wmax": 1.0}, {"g": g}),
                                  init_postsynaptic("ExpCurr", {"tau": 5.0}))
    sg.set_sparse_connections(pre, post)
    return m, steps, 100


def izhikevich():
    rng = np.random.default_rng(10)
    m = GeNNModel("float", "izhikevich")
    m.dt = 0.5
    n = 300
    pop = m.add_neuron_population("izh", n, "Izhikevich", {"a": 0.02, "b": 0.2, "c": -65.0, "d": 8.0},
                                  {"V": rng.uniform(-70, -60, n).astype(np.float32), "U": -13.0})
    m.add_current_source("drive", "DC", pop, {"amp": 6.0}, {})
    pop.spike_recording_enabled = True
    pre = rng.integers(0, n, size=6000).astype(np.uint32)
    post = rng.integers(0, n, size=6000).astype(np.uint32)
    g = rng.normal(0.5, 0.2, size=6000).astype(np.float32)
    sg = m.add_synapse_population("rec", "SPARSE", pop, pop, init_weight_update("StaticPulse", {}, {"g": g}),
                                  init_postsynaptic("DeltaCurr", {}))
    sg.set_sparse_connections(pre, post)
    return m, 400, 100


def poisson_drive():
    """Potjans architecture in miniature with its PoissonExp background drive.
    The draws come from the library's own Philox streams, so this case has no
    reference golden vector: it pins the CUDA kernels to the CPU checker
    (identical streams) and both to the reference statistically."""
    m = workloads.potjans(neuron_scale=0.01, seed=11, host_connectivity=True, background="poisson", record=True)
    return m, 300, 100


CASES = {"ff_sparse": ff_sparse, "c1_full": c1_full, "ff_sparse_narrow": ff_sparse_narrow, "ff_bitmask": ff_bitmask,
         "ff_dense": ff_dense, "potjans_mini": potjans_mini, "potjans_mini_d1": potjans_mini_d1, "cond_delay": cond_delay, "stdp": stdp,
         "izhikevich": izhikevich}


# ---------------------------------------------------------------------------
# Config-scale networks compared on population statistics (rates and CV-ISI over
# 10 s of simulated time): recurrent networks are chaotic, so two correct
# simulators agree on those, not spike by spike.  Each builder returns
# (GeNNModel, steps); connectivity, weights, delays and initial potentials are
# drawn on the host from the seed so that the reference's CPU backend and the
# CUDA kernels are loaded with identical arrays.
# ---------------------------------------------------------------------------
def stats_potjans_x1(shard=None):
    m = workloads.potjans(neuron_scale=1.0, seed=2024, host_connectivity=True, background="poisson", record=True,
                          shard=shard)
    return m, 100000


def stats_cond_ei(shard=None):
    m = workloads.cond_ei(neuron_scale=1.0, seed=4321, shard=shard)
    return m, 100000


STATS_CASES = {"potjans_x1": stats_potjans_x1, "cond_ei": stats_cond_ei}
