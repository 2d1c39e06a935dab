"""GPU parity: the CUDA kernels, called through the C ABI, against the
reference's golden vectors (tests/golden/, produced by the unmodified
single_threaded_cpu backend) and against the CPU checker on the same inputs.

Bars: spike (step, id) sets bit-exact; membrane state, postsynaptic input
buffers and learned weights within 1e-5 relative (fp32) with an absolute floor
for values near zero, because fp32 reductions into shared targets are unordered
on the GPU."""
import numpy as np
import pytest

from genn_b200.resolve import resolve
from tests import helpers
from tests.cases import CASES

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 2e-6

# the time-step paths: the persistent kernel in each of its schedules (spikes one step late where no synapse
# arrives in the same step; only the same-step synapses before the neuron update;
# everything before it; near synapses delivered by the spiking thread itself; the
# split schedule on the warp-specialised kernel and on the plain one); one launch per
# kernel.  (use_fused, use_lag, use_emit, use_split, stream_warps)
PATHS = {"persistent": (1, 1, 1, 1, -1), "persistent-emit": (1, 0, 1, 1, -1),
         "persistent-split": (1, 0, 0, 1, -1), "persistent-split-one-warp-set": (1, 0, 0, 1, 0),
         "persistent-plain": (1, 0, 0, 0, -1), "per-kernel": (0, 1, 1, 1, -1),
         # one launch per kernel with EVERY step delivered by the target-tiled kernel (shared-memory
         # accumulation over the private tile-major copy), which production takes only for heavy steps
         "per-kernel-tiled": (0, 1, 1, 1, -1),
         # the same with tickets of at most four synaptic events (one spike each, a ticket per run)
         "per-kernel-tiled-small-tickets": (0, 1, 1, 1, -1)}
# networks whose SPARSE groups the target-tiled kernel serves (non-learning)
TILED_CASES = {"ff_sparse", "c1_full", "ff_sparse_narrow", "potjans_mini", "potjans_mini_d1", "cond_delay", "izhikevich"}
# networks whose every synapse has a dendritic delay of at least one step
LAG_CASES = {"potjans_mini_d1"}
# networks with dendritic-delay rings (some of whose synapses may arrive in the same step)
RING_CASES = {"potjans_mini", "potjans_mini_d1"}


def _select(rt, path, name=None):
    fused, lag, emit, split, stream = PATHS[path]
    rt.set_option("use_fused", fused)
    rt.set_option("use_lag", lag)
    rt.set_option("use_emit", emit)
    rt.set_option("use_split", split)
    rt.set_option("stream_warps", stream)
    if path.startswith("per-kernel-tiled"):
        rt.set_option("tiled_min_events", 0)
        if path.endswith("small-tickets"):
            rt.set_option("tiled_ticket_events", 4)
        if name in TILED_CASES:
            assert rt.counter("tiled_ready") == 1 and rt.counter("tiled_synapses") > 0
    if name is not None and rt.step_path()[0] >= 1:
        want = (2 if (lag and name in LAG_CASES) else 3 if (emit and stream != 0 and name in RING_CASES)
                else 1 if (split and name in RING_CASES) else 0)
        assert rt.schedule == want, f"{name}: schedule {rt.schedule}, expected {want}"
        assert rt.lagging == (want == 2 and bool(fused))
        assert (rt.counter("stream_warps") > 0) == (want in (1, 3) and stream != 0), "warp-specialised kernel expected"


def _runtime(net, steps, **kw):
    from genn_b200.runtime import Runtime
    return Runtime(None, steps, net=net, **kw)


class _Adapter:
    """Gives the CUDA runtime the interface helpers.run_and_collect drives."""

    def __init__(self, rt):
        self.rt = rt

    def step(self, n):
        self.rt.step_time(n)

    def array(self, name):
        return self.rt.array(name)

    def current_spikes(self, pop):
        return self.rt.current_spikes(pop)


@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("name", list(CASES))
def test_step_by_step_matches_reference_golden(name, path):
    """Every time-step path (a model not eligible for a persistent kernel falls
    back to the next one, as in production)."""
    model, steps, dump_every = CASES[name]()
    net = resolve(model)
    rt = _runtime(net, steps)
    _select(rt, path, name)
    got = helpers.run_and_collect(_Adapter(rt), net, steps, dump_every)
    helpers.compare(got, helpers.load_golden(name), exact_state=False, rtol=RTOL, atol=ATOL)
    if path.startswith("per-kernel-tiled") and name in TILED_CASES:
        assert rt.counter("heavy") == 1, "the tiled kernel was meant to deliver every step"
    rt.close()


def test_tiled_kernels_are_armed_by_activity():
    """A threshold the network's steps reach: after a block of steps whose spike counts have arrived on the
    host the tiled kernels are launched, and the run still matches the reference fixture."""
    model, steps, dump_every = CASES["potjans_mini"]()
    net = resolve(model)
    rt = _runtime(net, steps)
    _select(rt, "per-kernel")
    rt.set_option("tiled_min_events", 200)
    assert rt.counter("tiled_ready") == 1 and rt.counter("tiled_armed") == 0
    got = helpers.run_and_collect(_Adapter(rt), net, steps, dump_every)
    helpers.compare(got, helpers.load_golden("potjans_mini"), exact_state=False, rtol=RTOL, atol=ATOL)
    # (single steps arm and disarm as spikes come and go; a block of 100 steps holds spikes for certain)
    rt.step_time(100)
    rt.synchronize()
    rt.step_time(1)
    assert rt.counter("tiled_armed") == 1, "the block's peak spike count was meant to arm the tiled kernels"
    rt.close()


def test_tiled_copy_follows_pushed_weights():
    """The tile-major copy is private: pushing new weights into the caller's array must reach it."""
    model, steps, _ = CASES["ff_sparse"]()
    net = resolve(model)
    outs = []
    for tiled in (1, 0):
        rt = _runtime(net, steps)
        _select(rt, "per-kernel-tiled" if tiled else "per-kernel")
        rt.step_time(20)
        rt.plan.push("syn.g", (net.syn("syn").g * 0.5).astype(np.float32))
        rt.step_time(80)
        outs.append((rt.array("psm0.out_post")[0], rt.array("post.V")[0]))
        rt.close()
    helpers.assert_close(outs[0][0], outs[1][0], "out_post after a weight push", RTOL, ATOL)
    helpers.assert_close(outs[0][1], outs[1][1], "V after a weight push", RTOL, ATOL)


@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("name", ["ff_sparse", "potjans_mini", "potjans_mini_d1", "cond_delay", "stdp"])
def test_many_steps_in_one_call_and_recording_match_reference_golden(name, path):
    """All steps in one call (one persistent launch, or replays of a captured
    graph) with spike recording on: the decoded recording equals the
    reference's spikes and the final state matches."""
    model, steps, dump_every = CASES[name]()
    net = resolve(model)
    rt = _runtime(net, steps)
    _select(rt, path, name)
    rt.set_option("graph_steps", 37)        # not a divisor of the step count: exercises the remainder path
    rt.step_time(steps)
    rt.synchronize()
    assert rt.timestep == steps
    rt.pull_recording_buffers()
    want = helpers.load_golden(name)
    for p in net.pops:
        if not p.record:
            continue
        times, ids = rt.recorded_spikes(p.name)[0]
        got = helpers.sorted_pairs(np.stack([np.rint(times / net.dt).astype(np.uint32), ids], axis=1))
        assert np.array_equal(got, want[f"spikes_{p.name}"]), f"recorded spikes of {p.name} differ"
    final = {k: v for k, v in helpers.snapshot(_Adapter(rt), net, steps).items()}
    helpers.compare(final, {k: v for k, v in want.items() if k.endswith(f"_{steps}")}, exact_state=False,
                    rtol=RTOL, atol=ATOL)
    rt.close()


@pytest.mark.parametrize("capacity", [None, 8])
def test_recording_pull_as_pairs_equals_the_recording(capacity):
    """The pull lists the recording's non-zero words on the device and fetches those; with no room
    for them it copies the arrays whole.  Either way the host sees the device's words."""
    model, steps, _ = CASES["potjans_mini"]()
    net = resolve(model)
    rt = _runtime(net, steps)
    rt.recording_pairs_capacity = capacity
    rt.step_time(steps)
    before = rt.factory.d2h_bytes
    rt.pull_recording_buffers()
    moved = rt.factory.d2h_bytes - before
    whole = 0
    for p in net.pops:
        if not p.record:
            continue
        device = rt.array(f"{p.name}.record")
        whole += device.nbytes
        assert np.array_equal(rt._recording_words(p.name), device), p.name
    assert (rt._rec_pairs is None) == (capacity is not None)
    assert moved < whole if capacity is None else moved >= whole
    rt.close()


@pytest.mark.parametrize("name,num", [("ff_sparse", 100), ("potjans_mini", 100), ("c1_full", 1000)])
def test_matches_cpu_checker_every_step(name, num):
    """Same inputs through the CPU checker (itself bit-identical to the reference on these
    networks): per-step postsynaptic input and membrane potential within tolerance at EVERY
    step, spikes identical.  `c1_full` is benchmark config 1 at its stated size, all 1000 steps.
    The tolerance on a summed input is relative to the sum of the magnitudes that went into it
    (inputs of opposite sign cancel, so the error scales with what was added, not with what is
    left)."""
    from oracle.oracle import OracleRunner
    model, steps, _ = CASES[name]()
    net = resolve(model)
    onet = resolve(CASES[name]()[0])
    rt, orc = _runtime(net, steps), OracleRunner(onet, steps)
    scales = helpers.ContributionScale(onet)
    for s in range(num):
        before = {p.name: orc.current_spikes(p.name) for p in onet.pops}
        rt.step_time(1)
        orc.step(1)
        scales.step(before)
        for p in net.pops:
            assert np.array_equal(np.sort(rt.current_spikes(p.name)), np.sort(orc.current_spikes(p.name))), \
                f"step {s}: spikes of {p.name} differ"
        for i in range(len(net.psms)):
            helpers.assert_close(rt.array(f"psm{i}.out_post")[0], orc.array(f"psm{i}.out_post")[0],
                                 f"step {s} psm{i}", RTOL, ATOL, scale=scales.scale(i))
        for p in net.pops:
            if p.kind == "LIF":
                helpers.assert_close(rt.array(f"{p.name}.V")[0], orc.array(f"{p.name}.V")[0],
                                     f"step {s} V {p.name}", RTOL, ATOL)
    rt.close()
    orc.close()


@pytest.mark.parametrize("path", list(PATHS))
def test_poisson_background_matches_cpu_checker(path):
    """PoissonExp background: the CPU checker replays the library's Philox
    streams, so spikes must be identical and state within tolerance."""
    from oracle.oracle import OracleRunner
    from tests.cases import poisson_drive
    model, steps, dump_every = poisson_drive()
    net, onet = resolve(model), resolve(poisson_drive()[0])
    rt, orc = _runtime(net, steps), OracleRunner(onet, steps)
    _select(rt, path, "potjans_mini")
    got = helpers.run_and_collect(_Adapter(rt), net, steps, dump_every)

    class O:
        step = staticmethod(lambda n: orc.step(n))
        array = staticmethod(lambda name: orc.array(name))
        current_spikes = staticmethod(lambda pop: orc.current_spikes(pop))
    want = helpers.run_and_collect(O, onet, steps, dump_every)
    assert sum(len(v) for k, v in want.items() if k.startswith("spikes_")) > 50
    helpers.compare(got, want, exact_state=False, rtol=RTOL, atol=ATOL)
    rt.close()
    orc.close()


def test_synaptic_event_counter():
    model, steps, _ = CASES["ff_sparse"]()
    net = resolve(model)
    rt = _runtime(net, steps)
    rt.set_option("count_events", 1)
    rt.step_time(steps)
    gold = helpers.load_golden("ff_sparse")
    sp = gold["spikes_pre"]
    rl = net.syn("syn").row_length
    assert rt.counter("synaptic_events") == int(rl[sp[sp[:, 0] < steps - 1][:, 1]].sum())
    rt.close()


def test_device_check_reports_bad_index():
    """An out-of-range postsynaptic index is skipped and reported, not dereferenced."""
    from genn_b200 import abi
    model, steps, _ = CASES["ff_sparse"]()
    net = resolve(model)
    bad = net.syn("syn")
    bad.ind = bad.ind.copy()
    bad.ind[:] = 100000
    with pytest.raises(abi.B200Error, match="out of range"):
        rt = _runtime(net, steps)           # the index check of the initialisation kernels may already catch it
        rt.step_time(50)
        rt.synchronize()


@pytest.mark.parametrize("name,schedule", [("potjans_mini_d1", 2), ("potjans_mini", 3), ("potjans_mini", 1)])
def test_launch_boundaries_of_every_schedule_leave_the_usual_state(name, schedule):
    """Persistent launches of odd lengths (spikes delivered one step late inside a
    launch, or only partly before the neuron update) alternate with steps on the
    per-kernel path: memory between launches must be what the plain schedule
    leaves, or the hand-over would lose or double-deliver spikes."""
    model, steps, dump_every = CASES[name]()
    net = resolve(model)
    rt = _runtime(net, steps)
    if schedule == 1:
        rt.set_option("use_emit", 0)
    assert rt.schedule == schedule
    done, chunk = 0, [1, 2, 1, 5, 3, 17, 1, 1, 40]
    i = 0
    while done < steps:
        n = min(chunk[i % len(chunk)], steps - done)
        rt.set_option("use_fused", 0 if (i % 3 == 2) else 1)
        rt.step_time(n)
        done += n
        i += 1
    rt.synchronize()
    rt.pull_recording_buffers()
    want = helpers.load_golden(name)
    for p in net.pops:
        if not p.record:
            continue
        times, ids = rt.recorded_spikes(p.name)[0]
        got = helpers.sorted_pairs(np.stack([np.rint(times / net.dt).astype(np.uint32), ids], axis=1))
        assert np.array_equal(got, want[f"spikes_{p.name}"]), f"recorded spikes of {p.name} differ"
    final = helpers.snapshot(_Adapter(rt), net, steps)
    helpers.compare(final, {k: v for k, v in want.items() if k.endswith(f"_{steps}")}, exact_state=False,
                    rtol=RTOL, atol=ATOL)
    rt.close()
