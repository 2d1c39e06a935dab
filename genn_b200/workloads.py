"""Seeded synthetic workloads with the shapes, sizes and value distributions of
the benchmark configurations.  Every builder returns a :class:`GeNNModel`
ready for ``build()``; inputs come from ``numpy.random.default_rng(seed)``.

The Potjans-Diesmann microcircuit parameters (population sizes, connection
probabilities, external in-degrees, weight and delay distributions) are the
ones tabulated in the reference's user project
(userproject/potjans_microcircuit.py:27-100); connectivity, weights, delays
and initial voltages are synthetic draws from those distributions.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import os

import numpy as np

from .model import (GeNNModel, init_postsynaptic, init_sparse_connectivity, init_var,
                    init_weight_update)


def poisson_spike_trains(rng, n: int, rate_hz: float, duration_ms: float):
    """Per-source sorted spike times: count ~ Poisson(rate*T), times ~ U[0,T).
    Returns (startSpike, endSpike, spikeTimes) as SpikeSourceArray wants them."""
    counts = rng.poisson(rate_hz * duration_ms / 1000.0, size=n)
    end = np.cumsum(counts).astype(np.uint32)
    start = (end - counts).astype(np.uint32)
    times = rng.uniform(0.0, duration_ms, size=int(end[-1]) if n else 0).astype(np.float32)
    for i in range(n):
        times[start[i]:end[i]].sort()
    return start, end, times


def truncated_normal(rng, mean: float, sd: float, lo: float, hi: float, size: int) -> np.ndarray:
    """Normal draws re-sampled until they fall inside [lo, hi], the semantics of
    the reference's NormalClipped snippets (initVarSnippet.h:163-172); fp32."""
    out = rng.standard_normal(size=size, dtype=np.float32)
    out *= np.float32(sd)
    out += np.float32(mean)
    bad = np.nonzero((out > hi) | (out < lo))[0]
    while len(bad):
        out[bad] = rng.standard_normal(size=len(bad), dtype=np.float32) * np.float32(sd) + np.float32(mean)
        bad = bad[(out[bad] > hi) | (out[bad] < lo)]
    return out


def feedforward(seed: int = 1, num_pre: int = 1000, num_post: int = 10000, prob: float = 0.1,
                rate_hz: float = 20.0, steps: int = 1000, dt: float = 0.1,
                matrix: str = "SPARSE", narrow: bool = False) -> GeNNModel:
    """Config 1: Poisson spike sources (host-generated trains) -> LIF through
    fixed-probability connectivity, fp32 weights U[0, 0.05) nA, ExpCurr."""
    rng = np.random.default_rng(seed)
    m = GeNNModel("float", "feedforward")
    m.dt = dt
    m.default_narrow_sparse_ind_enabled = narrow
    start, end, times = poisson_spike_trains(rng, num_pre, rate_hz, steps * dt)
    src = m.add_neuron_population("pre", num_pre, "SpikeSourceArray", {},
                                  {"startSpike": start, "endSpike": end})
    src.set_extra_global_param("spikeTimes", times)
    lif = {"C": 0.25, "TauM": 20.0, "Vrest": -65.0, "Vreset": -70.0, "Vthresh": -50.0,
           "Ioffset": 0.0, "TauRefrac": 2.0}
    trg = m.add_neuron_population("post", num_post, "LIF", lif, {"V": -65.0, "RefracTime": 0.0})
    src.spike_recording_enabled = True
    trg.spike_recording_enabled = True
    mask = rng.random((num_pre, num_post)) < prob
    pre, post = np.nonzero(mask)
    g = rng.uniform(0.0, 0.05, size=len(pre)).astype(np.float32)
    if matrix == "SPARSE":
        sg = m.add_synapse_population("syn", "SPARSE", src, trg,
                                      init_weight_update("StaticPulse", {}, {"g": g}),
                                      init_postsynaptic("ExpCurr", {"tau": 5.0}))
        sg.set_sparse_connections(pre, post)
    elif matrix == "BITMASK":
        sg = m.add_synapse_population("syn", "BITMASK", src, trg,
                                      init_weight_update("StaticPulseConstantWeight", {"g": 0.025}),
                                      init_postsynaptic("ExpCurr", {"tau": 5.0}))
        sg.set_sparse_connections(pre, post)
    elif matrix == "DENSE":
        dense = np.zeros((num_pre, num_post), dtype=np.float32)
        dense[pre, post] = g
        m.add_synapse_population("syn", "DENSE", src, trg,
                                 init_weight_update("StaticPulse", {}, {"g": dense}),
                                 init_postsynaptic("ExpCurr", {"tau": 5.0}))
    else:
        raise ValueError(matrix)
    return m


# ---------------------------------------------------------------------------
# Potjans-Diesmann microcircuit architecture
# ---------------------------------------------------------------------------
POTJANS_POPS = ["23E", "23I", "4E", "4I", "5E", "5I", "6E", "6I"]
POTJANS_NUM = {"23E": 20683, "23I": 5834, "4E": 21915, "4I": 5479,
               "5E": 4850, "5I": 1065, "6E": 14395, "6I": 2948}
# probability of >=1 connection; row = target, column = source (POTJANS_POPS order)
POTJANS_PROB = np.array([
    [0.1009, 0.1689, 0.0437, 0.0818, 0.0323, 0.0,    0.0076, 0.0],
    [0.1346, 0.1371, 0.0316, 0.0515, 0.0755, 0.0,    0.0042, 0.0],
    [0.0077, 0.0059, 0.0497, 0.135,  0.0067, 0.0003, 0.0453, 0.0],
    [0.0691, 0.0029, 0.0794, 0.1597, 0.0033, 0.0,    0.1057, 0.0],
    [0.1004, 0.0622, 0.0505, 0.0057, 0.0831, 0.3726, 0.0204, 0.0],
    [0.0548, 0.0269, 0.0257, 0.0022, 0.06,   0.3158, 0.0086, 0.0],
    [0.0156, 0.0066, 0.0211, 0.0166, 0.0572, 0.0197, 0.0396, 0.2252],
    [0.0364, 0.001,  0.0034, 0.0005, 0.0277, 0.008,  0.0658, 0.1443]])
POTJANS_EXT = {"23E": 1600, "23I": 1500, "4E": 2100, "4I": 1900,
               "5E": 2000, "5I": 1900, "6E": 2900, "6I": 2100}
POTJANS_BG_RATE = 8.0
POTJANS_MEAN_W = 87.8e-3
POTJANS_G = -4.0
POTJANS_DELAY = {"E": (1.5, 0.75), "I": (0.75, 0.375)}
# 0.9999 quantile of the standard normal (scipy.stats.norm.ppf(0.9999))
_NORMAL_Q9999 = 3.719016485455709


def potjans_in_degree(src: str, trg: str) -> int:
    """Full-scale in-degree of ``trg`` from ``src``: total synapses for the
    pairwise connection probability, divided by the target count."""
    ns, nt = POTJANS_NUM[src], POTJANS_NUM[trg]
    p = POTJANS_PROB[POTJANS_POPS.index(trg), POTJANS_POPS.index(src)]
    if p == 0.0:
        return 0
    total = int(round(math.log(1.0 - p) / math.log(float(nt * ns - 1) / float(nt * ns))))
    return total // nt


def potjans_max_delay_slots(dt: float = 0.1) -> int:
    mx = max(m + s * _NORMAL_Q9999 for m, s in POTJANS_DELAY.values())
    return int(round(mx / dt))


def potjans_projections(neuron_scale: float = 1.0):
    """[(src, trg, num_synapses, mean_w, sd_w, mean_d, sd_d, max_d)] for the
    non-empty projections; in-degree fixed, neuron counts scaled."""
    out = []
    for trg in POTJANS_POPS:
        for src in POTJANS_POPS:
            k = potjans_in_degree(src, trg)
            nt = int(round(neuron_scale * POTJANS_NUM[trg]))
            num = int(round(k * float(nt)))
            if num <= 0:
                continue
            if src.endswith("E"):
                mean_w = 2.0 * POTJANS_MEAN_W if (src == "4E" and trg == "23E") else POTJANS_MEAN_W
            else:
                mean_w = POTJANS_G * POTJANS_MEAN_W
            sd_w = mean_w * 0.05 if (src == "4E" and trg == "23E") else abs(mean_w * 0.1)
            md, sd = POTJANS_DELAY[src[-1]]
            out.append((src, trg, num, mean_w, sd_w, md, sd, md + sd * _NORMAL_Q9999))
    return out


def potjans(neuron_scale: float = 1.0, seed: int = 1234, dt: float = 0.1,
            host_connectivity: bool = False, background: str = "poisson",
            shard: Optional[Tuple[int, int]] = None, record: bool = False,
            min_delay: float = 0.0, extra_delay_slots: int = 0) -> GeNNModel:
    """Potjans-Diesmann microcircuit architecture at ``neuron_scale`` times the
    published population sizes with the published in-degrees.

    ``min_delay`` (ms) is the lower clip of the delay distribution: 0 as in the
    reference's script (userproject/potjans_microcircuit.py:259), which rounds a
    few per cent of the synapses to a delay of zero steps; ``dt`` gives every
    synapse at least one step, as in the original model description.
    ``extra_delay_slots`` lengthens the dendritic-delay ring beyond the script's
    round(longest delay / dt): with exactly that many slots a synapse drawn at
    the longest delay wraps around the ring and arrives in the same step.

    ``host_connectivity`` draws connectivity/weights/delays with numpy so the
    same arrays can be handed to a CPU checker (small scales only); otherwise
    they are drawn on the GPU by the initialisation kernels from the same
    distributions.  ``background`` is "poisson" (PoissonExp current source at
    8 Hz x external in-degree) or "dc" (its mean as a constant current, for
    RNG-free comparisons).  ``shard=(rank, world)`` keeps only the synapses
    whose postsynaptic neuron lies in this rank's contiguous slice of each
    population.
    """
    rng = np.random.default_rng(seed)
    m = GeNNModel("float", "potjans_microcircuit")
    m.dt = dt
    m.seed = seed
    m.fuse_postsynaptic_models = True
    m.default_narrow_sparse_ind_enabled = True
    slots = potjans_max_delay_slots(dt)
    pops = {}
    for name in POTJANS_POPS:
        n = int(round(neuron_scale * POTJANS_NUM[name]))
        lif = {"C": 0.25, "TauM": 10.0, "Vrest": -65.0, "Vreset": -65.0, "Vthresh": -50.0,
               "Ioffset": 0.0, "TauRefrac": 2.0}
        rate = POTJANS_EXT[name] * POTJANS_BG_RATE
        if background == "dc":
            # mean of the filtered Poisson drive: weight * rate[kHz] * tauSyn
            lif["Ioffset"] = POTJANS_MEAN_W * (rate / 1000.0) * 0.5
        v0 = (rng.normal(-58.0, 5.0, size=n).astype(np.float32) if host_connectivity
              else init_var("Normal", {"mean": -58.0, "sd": 5.0}))
        pop = m.add_neuron_population(name, n, "LIF", lif, {"V": v0, "RefracTime": 0.0})
        if background == "poisson":
            m.add_current_source(name + "_poisson", "PoissonExp", pop,
                                 {"weight": POTJANS_MEAN_W, "tauSyn": 0.5, "rate": rate}, {"current": 0.0})
        pop.spike_recording_enabled = record
        pops[name] = pop
    drawn = {}
    if host_connectivity:
        # every projection has a random stream of its own (seed, projection index), so the projections
        # can be drawn side by side: numpy releases the interpreter lock inside its generators
        from concurrent.futures import ThreadPoolExecutor
        projections = list(potjans_projections(neuron_scale))

        def draw(index):
            src, trg, num, mean_w, sd_w, md, sd, mxd = projections[index]
            ns, nt = pops[src].num_neurons, pops[trg].num_neurons
            lo, hi = (0.0, float(np.finfo(np.float32).max)) if mean_w > 0 else (-float(np.finfo(np.float32).max), 0.0)
            prng = np.random.default_rng([seed, 1000 + index])
            # `num` synapses placed uniformly with replacement (FixedNumberTotalWithReplacement): the row
            # lengths are multinomial; drawing them first gives the pairs row by row without a sort
            counts = prng.multinomial(num, np.full(ns, 1.0 / ns))
            pre = np.repeat(np.arange(ns, dtype=np.uint32), counts)
            post = prng.integers(0, nt, size=num, dtype=np.uint32)
            g = truncated_normal(prng, mean_w, sd_w, lo, hi, num)
            # NormalClippedDelay: truncated normal in time steps, then rint
            d = truncated_normal(prng, md / dt, sd / dt, min_delay / dt, mxd / dt, num)
            np.rint(d, out=d)
            d = d.astype(np.uint8)
            if shard is not None:
                from .plan import shard_bounds
                bounds = shard_bounds(nt, shard[1])
                keep = (post >= bounds[shard[0]]) & (post < bounds[shard[0] + 1])
                pre, post, g, d = pre[keep], post[keep], g[keep], d[keep]
            return pre, post, g, d

        with ThreadPoolExecutor(max_workers=max(1, min(16, os.cpu_count() or 1))) as pool:
            drawn = dict(enumerate(pool.map(draw, range(len(projections)))))
    for index, (src, trg, num, mean_w, sd_w, md, sd, mxd) in enumerate(potjans_projections(neuron_scale)):
        ns, nt = pops[src].num_neurons, pops[trg].num_neurons
        lo, hi = (0.0, float(np.finfo(np.float32).max)) if mean_w > 0 else (-float(np.finfo(np.float32).max), 0.0)
        if host_connectivity:
            pre, post, g, d = drawn.pop(index)
            wu = init_weight_update("StaticPulseDendriticDelay", {}, {"g": g, "d": d})
            sg = m.add_synapse_population(f"{src}_{trg}", "SPARSE", pops[src], pops[trg], wu,
                                          init_postsynaptic("ExpCurr", {"tau": 0.5}))
            sg.set_sparse_connections(pre, post, presorted=True)
        else:
            trg_range = None
            if shard is not None:
                # this process draws only the sub-matrix onto its own slice of the
                # targets: same in-degree, so its share of the synapses
                from .plan import shard_bounds
                rank, world = shard
                bounds = shard_bounds(nt, world)
                trg_range = (bounds[rank], bounds[rank + 1])
                num = int(round(num * (trg_range[1] - trg_range[0]) / float(nt)))
            wu = init_weight_update("StaticPulseDendriticDelay", {}, {
                "g": init_var("NormalClipped", {"mean": mean_w, "sd": sd_w, "min": lo, "max": hi}),
                "d": init_var("NormalClippedDelay", {"mean": md, "sd": sd, "min": min_delay, "max": mxd})})
            sg = m.add_synapse_population(
                f"{src}_{trg}", "SPARSE", pops[src], pops[trg], wu,
                init_postsynaptic("ExpCurr", {"tau": 0.5}),
                init_sparse_connectivity("FixedNumberTotalWithReplacement", {"num": num}))
            sg.trg_range = trg_range
        sg.max_dendritic_delay_timesteps = slots + extra_delay_slots
    return m


# ---------------------------------------------------------------------------
# Recurrent conductance-based E/I network (config 2)
# ---------------------------------------------------------------------------
def cond_ei(neuron_scale: float = 1.0, seed: int = 4321, dt: float = 0.1, in_degree: int = 1000,
            i_offset: float = 0.35, record: bool = True,
            shard: Optional[Tuple[int, int]] = None) -> GeNNModel:
    """80 000 excitatory + 20 000 inhibitory LIF neurons (times ``neuron_scale``)
    with a fixed in-degree: every neuron draws ``in_degree`` presynaptic partners
    uniformly (with replacement) from the whole network.  Constant weights
    0.6 nS (excitatory) and 6.7 nS (inhibitory), exponential conductances with
    tau 5 / 10 ms and reversal 0 / -80 mV, 1 ms axonal delay, initial potentials
    U[-60, -50) mV.  Conductances are in uS (potentials in mV, currents in nA, as
    in neuronModels.h:225-256).  ``i_offset`` is the constant current that keeps
    the network firing (the published description names no drive; without one
    every potential decays to rest).  Connectivity is drawn on the host so that
    a CPU checker can be handed identical arrays."""
    rng = np.random.default_rng(seed)
    m = GeNNModel("float", "cond_ei")
    m.dt = dt
    m.seed = seed
    ne, ni = int(round(80000 * neuron_scale)), int(round(20000 * neuron_scale))
    lif = {"C": 0.2, "TauM": 20.0, "Vrest": -60.0, "Vreset": -60.0, "Vthresh": -50.0, "Ioffset": i_offset,
           "TauRefrac": 5.0}
    pops = {}
    for name, n in (("E", ne), ("I", ni)):
        v0 = rng.uniform(-60.0, -50.0, size=n).astype(np.float32)
        pops[name] = m.add_neuron_population(name, n, "LIF", lif, {"V": v0, "RefracTime": 0.0})
        pops[name].spike_recording_enabled = record
    delay_steps = int(round(1.0 / dt))
    for trg_name, nt in (("E", ne), ("I", ni)):
        lo, hi = 0, nt
        if shard is not None:
            from .plan import shard_bounds
            bounds = shard_bounds(nt, shard[1])
            lo, hi = bounds[shard[0]], bounds[shard[0] + 1]
        # one stream of draws per target population, the same on every rank
        pre_all = rng.integers(0, ne + ni, size=(nt, in_degree), dtype=np.int64)[lo:hi]
        post_all = np.repeat(np.arange(lo, hi, dtype=np.uint32), in_degree)
        pre_all = pre_all.reshape(-1)
        for src_name, w, tau, erev in (("E", 0.6e-3, 5.0, 0.0), ("I", 6.7e-3, 10.0, -80.0)):
            sel = (pre_all < ne) if src_name == "E" else (pre_all >= ne)
            pre = (pre_all[sel] - (0 if src_name == "E" else ne)).astype(np.uint32)
            sg = m.add_synapse_population(f"{src_name}{trg_name}", "SPARSE", pops[src_name], pops[trg_name],
                                          init_weight_update("StaticPulseConstantWeight", {"g": w}),
                                          init_postsynaptic("ExpCond", {"tau": tau, "E": erev}))
            sg.set_sparse_connections(pre, post_all[sel])
            sg.axonal_delay_steps = delay_steps
    return m


# ---------------------------------------------------------------------------
# PROCEDURAL connectivity stress test (config 4)
# ---------------------------------------------------------------------------
def procedural_stress(num_neurons: int = 1_000_000, prob: float = 0.001, driven_fraction: float = 0.1,
                      drive_rate_hz: float = 5.0, threads_per_spike: int = 32, seed: int = 77,
                      dt: float = 1.0, record: bool = False) -> GeNNModel:
    """``num_neurons`` LIF neurons, recurrently connected with probability ``prob`` through PROCEDURAL
    connectivity: no synapse is stored, every spike regenerates its row (about ``prob * num_neurons``
    targets) and the weights (Normal, mean 0.1 nA, sd 0.01) from Philox streams keyed on the seed and
    the presynaptic index.  ``driven_fraction`` of the neurons receive a Poisson drive of
    ``drive_rate_hz`` (one PoissonExp source each, strong enough that every drive event makes a spike);
    they form a population of their own, so the network has 2 x 2 recurrent projections.
    ``threads_per_spike`` threads share each row.  Purely excitatory: the network runs up to the rate
    its refractory period allows, which is what a stress test of the regeneration path wants."""
    m = GeNNModel("float", "procedural_stress")
    m.dt = dt
    m.seed = seed
    lif = {"C": 0.25, "TauM": 20.0, "Vrest": -65.0, "Vreset": -70.0, "Vthresh": -50.0, "Ioffset": 0.0, "TauRefrac": 5.0}
    n_driven = int(round(num_neurons * driven_fraction))
    pops = {}
    for name, n in (("driven", n_driven), ("rest", num_neurons - n_driven)):
        if n == 0:
            continue
        pops[name] = m.add_neuron_population(name, n, "LIF", lif, {"V": init_var("Uniform", {"min": -65.0, "max": -55.0}),
                                                                   "RefracTime": 0.0})
        pops[name].spike_recording_enabled = record
    if "driven" in pops:
        m.add_current_source("drive", "PoissonExp", pops["driven"], {"weight": 1.0, "tauSyn": 5.0, "rate": drive_rate_hz},
                             {"current": 0.0})
    for a in pops:
        for b in pops:
            sg = m.add_synapse_population(f"{a}_{b}", "PROCEDURAL", pops[a], pops[b],
                                          init_weight_update("StaticPulse", {}, {"g": init_var("Normal", {"mean": 0.1, "sd": 0.01})}),
                                          init_postsynaptic("ExpCurr", {"tau": 5.0}),
                                          init_sparse_connectivity("FixedProbability", {"prob": prob}))
            sg.num_threads_per_spike = threads_per_spike
    return m


# ---------------------------------------------------------------------------
# Batched plasticity (config 5)
# ---------------------------------------------------------------------------
def batched_stdp(num_pre: int = 10000, num_post: int = 10000, prob: float = 0.1, batch: int = 32,
                 rate_hz: float = 25.0, seed: int = 55, dt: float = 1.0, world: int = 1):
    """``num_pre`` Poisson inputs -> ``num_post`` LIF neurons through SPARSE fixed-probability
    connectivity with pair-based additive STDP (tau+ = tau- = 20 ms,
    A+ = 0.01, A- = 0.0105, weights clipped to [0, 1] nA, initial weights U[0, 0.5)); ``batch``
    independent copies of the dynamic state per process, every copy with its own weights.  The custom
    update group "gradient" sums the weights over the batch (and, in a data-parallel run of ``world``
    processes, over the processes) and writes the mean back into every copy.  Every input fires at
    ``rate_hz`` (the mean of the published U[0, 50) Hz: the Poisson model here has one rate per
    population), drawn independently per batch entry.  Returns (model, synapse group)."""
    m = GeNNModel("float", "batched_stdp")
    m.dt = dt
    m.seed = seed
    m.batch_size = batch
    src = m.add_neuron_population("input", num_pre, "Poisson", {"rate": rate_hz}, {"timeStepToSpike": 0.0})
    # (the published description gives no neuron constants; with 1 000 inputs of up to 1 nA each a membrane
    # capacitance of 40 nF keeps the outputs at tens of Hz instead of at the limit their refractory period sets)
    lif = {"C": 40.0, "TauM": 20.0, "Vrest": -65.0, "Vreset": -70.0, "Vthresh": -55.0, "Ioffset": 0.0, "TauRefrac": 2.0}
    trg = m.add_neuron_population("output", num_post, "LIF", lif, {"V": init_var("Uniform", {"min": -70.0, "max": -56.0}),
                                                                   "RefracTime": 0.0})
    # (connectivity and initial weights drawn on the host: the column-major view that the postsynaptic half of
    # STDP walks is built from host-supplied rows)
    rng = np.random.default_rng(seed)
    pre, post = np.nonzero(rng.random((num_pre, num_post), dtype=np.float32) < prob)
    g = rng.uniform(0.0, 0.5, size=len(pre)).astype(np.float32)
    sg = m.add_synapse_population("syn", "SPARSE", src, trg,
                                  init_weight_update("STDP", {"tauPlus": 20.0, "tauMinus": 20.0, "Aplus": 0.01, "Aminus": 0.0105,
                                                              "Wmin": 0.0, "Wmax": 1.0}, {"g": g}),
                                  init_postsynaptic("ExpCurr", {"tau": 5.0}))
    sg.set_sparse_connections(pre.astype(np.uint32), post.astype(np.uint32), presorted=True)
    m.add_custom_update("mean_g", "gradient", "SUM", (sg, "g"), broadcast=True, scale=1.0 / (batch * world))
    return m, sg
