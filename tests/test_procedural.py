"""PROCEDURAL connectivity (presynapticUpdateStrategySIMT.cc:394-566): nothing of
the matrix is stored, rows and weights are regenerated for every spike.

The reference regenerates them from its own random streams, which only CUDA
builds have, so there is no reference fixture for this path.  What is checked:
the regenerated matrix is EXACTLY the one the initialisation kernels store for
a SPARSE group with the same snippets and streams (the two runs must agree on
every spike and, up to the order of fp32 additions, on every variable), and that
stored matrix, pulled back and handed to the CPU checker, gives the same run."""
import numpy as np
import pytest

from genn_b200 import GeNNModel, init_postsynaptic, init_sparse_connectivity, init_var, init_weight_update
from genn_b200.resolve import resolve
from genn_b200.workloads import poisson_spike_trains
from tests import helpers

pytestmark = pytest.mark.gpu
STEPS = 400


def _model(matrix, stored=None):
    """Spike sources -> LIF through a fixed-probability group with drawn weights and a
    fixed-out-degree group with one constant negative weight.  `stored`: {group: (pre, post, g)}
    builds the same network from explicit synapse lists instead."""
    rng = np.random.default_rng(11)
    m = GeNNModel("float", "procedural")
    m.dt = 0.1
    m.seed = 4321
    start, end, times = poisson_spike_trains(rng, 300, 80.0, STEPS * m.dt)
    pre = m.add_neuron_population("pre", 300, "SpikeSourceArray", {}, {"startSpike": start, "endSpike": end})
    pre.set_extra_global_param("spikeTimes", times)
    lif = {"C": 0.25, "TauM": 20.0, "Vrest": -65.0, "Vreset": -70.0, "Vthresh": -50.0, "Ioffset": 0.1, "TauRefrac": 2.0}
    post = m.add_neuron_population("post", 700, "LIF", lif, {"V": -65.0, "RefracTime": 0.0})
    post.spike_recording_enabled = True
    if stored is None:
        m.add_synapse_population("exc", matrix, pre, post,
                                 init_weight_update("StaticPulse", {}, {"g": init_var("Uniform", {"min": 0.0, "max": 0.08})}),
                                 init_postsynaptic("ExpCurr", {"tau": 5.0}),
                                 init_sparse_connectivity("FixedProbability", {"prob": 0.12}))
        m.add_synapse_population("inh", matrix, pre, post,
                                 init_weight_update("StaticPulseConstantWeight", {"g": -0.01}),
                                 init_postsynaptic("ExpCurr", {"tau": 8.0}),
                                 init_sparse_connectivity("FixedNumberPostWithReplacement", {"num": 25}))
    else:
        p, q, g = stored["exc"]
        sg = m.add_synapse_population("exc", "SPARSE", pre, post, init_weight_update("StaticPulse", {}, {"g": g}),
                                      init_postsynaptic("ExpCurr", {"tau": 5.0}))
        sg.set_sparse_connections(p, q)
        p, q, _ = stored["inh"]
        sg = m.add_synapse_population("inh", "SPARSE", pre, post, init_weight_update("StaticPulseConstantWeight", {"g": -0.01}),
                                      init_postsynaptic("ExpCurr", {"tau": 8.0}))
        sg.set_sparse_connections(p, q)
    return m


def _stored_lists(rt, net):
    out = {}
    for s in net.syns:
        rl = rt.array(f"{s.name}.row_length")
        ind = rt.array(f"{s.name}.ind").reshape(len(rl), s.row_stride)
        keep = np.arange(s.row_stride)[None, :] < rl[:, None]
        pre = np.repeat(np.arange(len(rl), dtype=np.uint32), rl)
        g = None
        if f"{s.name}.g" in rt.plan.arrays:
            g = rt.array(f"{s.name}.g").reshape(len(rl), s.row_stride)[keep]
        out[s.name] = (pre, ind[keep].astype(np.uint32), g)
    return out


def test_regenerated_matrix_is_the_stored_one_and_matches_the_cpu_checker():
    from genn_b200.runtime import Runtime
    from oracle.oracle import OracleRunner
    net_p, net_s = resolve(_model("PROCEDURAL")), resolve(_model("SPARSE"))
    rt_p, rt_s = Runtime(None, STEPS, net=net_p), Runtime(None, STEPS, net=net_s)
    assert rt_p.step_path()[0] == 0, "procedural groups run on the one-launch-per-kernel path"
    assert "exc.ind" not in rt_p.plan.arrays and "exc.g" not in rt_p.plan.arrays, "nothing of the matrix may be stored"
    stored = _stored_lists(rt_s, net_s)
    assert 0.10 < len(stored["exc"][0]) / (300 * 700) < 0.14
    assert len(stored["inh"][0]) == 300 * 25
    orc = OracleRunner(resolve(_model("SPARSE", stored)), STEPS)
    spikes = 0
    for step in range(STEPS):
        rt_p.step_time(1)
        rt_s.step_time(1)
        orc.step(1)
        a, b, c = (np.sort(x.current_spikes("post")) for x in (rt_p, rt_s, orc))
        assert np.array_equal(a, b) and np.array_equal(a, c), f"step {step}: spikes differ"
        spikes += len(a)
        if step % 50 == 49:
            for name in ("post.V", "psm0.out_post", "psm1.out_post"):
                helpers.assert_close(rt_p.array(name)[0], rt_s.array(name)[0], f"step {step} {name} vs stored", 1e-5, 2e-6)
                helpers.assert_close(rt_p.array(name)[0], orc.array(name)[0], f"step {step} {name} vs checker", 1e-5, 2e-6)
    assert spikes > 100
    # the event counters agree too: every regenerated synapse was delivered
    rt_p.close(); rt_s.close(); orc.close()


def test_many_steps_in_one_call():
    from genn_b200.runtime import Runtime
    net_p, net_s = resolve(_model("PROCEDURAL")), resolve(_model("SPARSE"))
    rt_p, rt_s = Runtime(None, STEPS, net=net_p), Runtime(None, STEPS, net=net_s)
    for rt in (rt_p, rt_s):
        rt.set_option("count_events", 1)
        rt.step_time(STEPS)
        rt.synchronize()
        rt.pull_recording_buffers()
    (ta, ia), (tb, ib) = rt_p.recorded_spikes("post")[0], rt_s.recorded_spikes("post")[0]
    assert np.array_equal(ia, ib) and np.allclose(ta, tb)
    assert rt_p.counter("synaptic_events") == rt_s.counter("synaptic_events") > 0
    rt_p.close(); rt_s.close()
