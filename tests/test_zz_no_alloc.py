"""The allocation-free neuron update (b200_update_neurons_noalloc) against the
regular entry point.

Some users of the library cannot call cudaMalloc while they run: a real-time
loop driving hardware from a spiking model, or a plugin with a memory budget
fixed at start-up.  The entry point under test keeps its
descriptor tables and counters in a fixed array inside the library instead.
Here two identical networks are advanced two steps, one through
b200_update_neurons and one through the new call (on a stream of its own), and
every array the update touches must come out the same, on both calls: the
second call reuses the scratch array the first one left behind.

This file is collected last on purpose, so a run that stops at the first failure
has already run everything else."""
import ctypes as C

import numpy as np
import pytest

from genn_b200 import abi
from genn_b200.resolve import resolve
from tests import helpers
from tests.cases import poisson_drive

pytestmark = pytest.mark.gpu


def _fresh():
    from genn_b200.runtime import Runtime
    model, steps, _ = poisson_drive()
    net = resolve(model)
    return net, Runtime(None, None, net=net)


def _touched_arrays(net):
    names = []
    for p in net.pops:
        names += [f"{p.name}.V", f"{p.name}.RefracTime", f"{p.name}.spk_cnt", f"{p.name}.spk"]
    for c in net.css:
        names.append(f"{c.name}.current")
    for i, psm in enumerate(net.psms):
        names.append(f"psm{i}.out_post")
        if psm.max_den_delay:
            names.append(f"psm{i}.den_delay")
    return names


def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row():
    import torch
    lib = abi.load_library()
    net_a, regular = _fresh()
    net_b, static = _fresh()
    # give the update something to consume: a pattern in every dendritic-delay ring
    rng = np.random.default_rng(3)
    for i, psm in enumerate(net_a.psms):
        if psm.max_den_delay:
            shape = regular.plan.arrays[f"psm{i}.den_delay"].shape
            ring = rng.normal(0.0, 0.05, size=shape).astype(np.float32)
            regular.plan.push(f"psm{i}.den_delay", ring)
            static.plan.push(f"psm{i}.den_delay", ring)
    regular.synchronize()
    static.synchronize()

    stream = torch.cuda.Stream()
    descs = (abi.NeuronGroupDesc * len(static.plan.neuron_descs))(*static.plan.neuron_descs)
    spikes_seen = 0
    for step in range(2):
        regular.update_neurons()
        rc = lib.b200_update_neurons_noalloc(0, C.c_void_p(stream.cuda_stream), descs, len(descs), 1, net_b.dt,
                                             net_b.seed, step, step, 0)
        assert rc == 0, lib.b200_noalloc_last_error().decode()
        torch.cuda.synchronize()
        regular.synchronize()
        for name in _touched_arrays(net_a):
            got, want = static.array(name), regular.array(name)
            if name.endswith(".spk"):
                # compare the slot this step wrote, as sets (emission order is not fixed)
                pop = name[:-4]
                slots = net_a.pop(pop).runtime_slots
                slot = (step + 1) % slots
                n = int(regular.array(f"{pop}.spk_cnt")[0, slot])
                assert n == int(static.array(f"{pop}.spk_cnt")[0, slot]), f"step {step}: spike count of {pop}"
                assert np.array_equal(np.sort(got[0, slot, :n]), np.sort(want[0, slot, :n])), f"step {step}: {name}"
                spikes_seen += n
            elif got.dtype == np.float32:
                helpers.assert_close(got.reshape(-1), want.reshape(-1), f"step {step}: {name}", 1e-5, 2e-6)
            else:
                assert np.array_equal(got, want), f"step {step}: {name}"
    assert spikes_seen > 0, "the case must produce spikes for the comparison to mean anything"
    regular.close()
    static.close()


def _batched_net(batch=2):
    """The Potjans miniature with its Poisson background, two batch elements, every synaptic
    weight zero: the CPU checker's time step (synapses, then neurons) then does to the state
    exactly what a neuron update alone does."""
    from genn_b200 import workloads
    m = workloads.potjans(neuron_scale=0.01, seed=11, host_connectivity=True, background="poisson", record=True)
    m.batch_size = batch
    net = resolve(m)
    for s in net.syns:
        s.g[...] = 0.0
    return net


def test_noalloc_matches_the_cpu_checker_with_recording_and_two_batch_elements():
    import torch
    from genn_b200.runtime import Runtime
    from oracle.oracle import OracleRunner
    lib = abi.load_library()
    steps, batch = 2, 2
    net = _batched_net(batch)
    static = Runtime(None, steps, net=net)
    orc = OracleRunner(_batched_net(batch), steps)
    rng = np.random.default_rng(5)
    for i, psm in enumerate(net.psms):
        if psm.max_den_delay:
            ring = rng.normal(0.2, 0.3, size=static.plan.arrays[f"psm{i}.den_delay"].shape).astype(np.float32)
            static.plan.push(f"psm{i}.den_delay", ring)
            orc.plan.push(f"psm{i}.den_delay", ring)
    static.synchronize()
    descs = (abi.NeuronGroupDesc * len(static.plan.neuron_descs))(*static.plan.neuron_descs)
    stream = torch.cuda.Stream()
    spikes_seen = 0
    for step in range(steps):
        orc.step(1)
        rc = lib.b200_update_neurons_noalloc(0, C.c_void_p(stream.cuda_stream), descs, len(descs), batch, net.dt,
                                             net.seed, step, step, steps)
        assert rc == 0, lib.b200_noalloc_last_error().decode()
        assert lib.b200_noalloc_check(0, C.c_void_p(stream.cuda_stream)) == 0, lib.b200_noalloc_last_error().decode()
        for name in _touched_arrays(net):
            got, want = static.array(name), orc.array(name)
            if name.endswith(".spk"):
                pop = name[:-4]
                slot = (step + 1) % net.pop(pop).runtime_slots
                for b in range(batch):
                    n = int(orc.array(f"{pop}.spk_cnt")[b, slot])
                    assert n == int(static.array(f"{pop}.spk_cnt")[b, slot]), f"step {step}: spike count of {pop}[{b}]"
                    assert np.array_equal(np.sort(got[b, slot, :n]), np.sort(want[b, slot, :n])), f"step {step}: {name}[{b}]"
                    spikes_seen += n
            elif got.dtype == np.float32:
                helpers.assert_close(got.reshape(-1), want.reshape(-1), f"step {step}: {name}", 1e-5, 2e-6)
            else:
                assert np.array_equal(got, want), f"step {step}: {name}"
    for p in net.pops:
        assert np.array_equal(static.array(f"{p.name}.record"), orc.array(f"{p.name}.record")), f"recording of {p.name}"
    assert spikes_seen > 0
    static.close()
    orc.close()


def test_noalloc_check_reports_a_spike_list_that_is_too_short():
    """A list stride smaller than the number of spikes of the step: the kernel drops the surplus
    (nothing is written out of bounds) and sets its check word, which b200_noalloc_check reports;
    the next update starts clean."""
    lib = abi.load_library()
    net, rt = _fresh()
    # every neuron above threshold: the whole population spikes in the step
    for p in net.pops:
        rt.plan.push(f"{p.name}.V", np.full(rt.plan.arrays[f"{p.name}.V"].shape, -40.0, dtype=np.float32))
    rt.synchronize()
    short = [abi.NeuronGroupDesc.from_buffer_copy(d) for d in rt.plan.neuron_descs]
    for d in short:
        d.spk_slot_stride = 4
    descs = (abi.NeuronGroupDesc * len(short))(*short)
    assert lib.b200_update_neurons_noalloc(0, None, descs, len(descs), 1, net.dt, net.seed, 0, 0, 0) == 0
    assert lib.b200_noalloc_check(0, None) == abi.ERR_DEVICE_CHECK
    assert b"spike list" in lib.b200_noalloc_last_error()
    # potentials were reset by the spikes: the same call again stays within the lists
    for p in net.pops:
        rt.plan.push(f"{p.name}.V", np.full(rt.plan.arrays[f"{p.name}.V"].shape, -65.0, dtype=np.float32))
    rt.synchronize()
    full = (abi.NeuronGroupDesc * len(short))(*rt.plan.neuron_descs)
    assert lib.b200_update_neurons_noalloc(0, None, full, len(full), 1, net.dt, net.seed, 1, 1, 0) == 0
    assert lib.b200_noalloc_check(0, None) == 0, lib.b200_noalloc_last_error().decode()
    rt.close()


def test_noalloc_refuses_a_stream_that_is_being_captured():
    import torch
    lib = abi.load_library()
    net, rt = _fresh()
    descs = (abi.NeuronGroupDesc * len(rt.plan.neuron_descs))(*rt.plan.neuron_descs)
    # the first call on the device (address look-up) comes before any capture
    assert lib.b200_update_neurons_noalloc(0, None, descs, len(descs), 1, net.dt, net.seed, 0, 0, 0) == 0
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        graph.capture_begin()
        try:
            rc = lib.b200_update_neurons_noalloc(0, C.c_void_p(stream.cuda_stream), descs, len(descs), 1, net.dt,
                                                 net.seed, 1, 1, 0)
        finally:
            graph.capture_end()
    assert rc == abi.ERR_STATE
    assert b"captured" in lib.b200_noalloc_last_error()
    rt.close()


def test_noalloc_rejects_more_groups_than_the_scratch_holds():
    lib = abi.load_library()
    net, rt = _fresh()
    too_many = 65
    descs = (abi.NeuronGroupDesc * too_many)(*([rt.plan.neuron_descs[0]] * too_many))
    rc = lib.b200_update_neurons_noalloc(0, None, descs, too_many, 1, net.dt, net.seed, 0, 0, 0)
    assert rc != 0
    assert b"exceed the limit of 64" in lib.b200_noalloc_last_error()
    rt.close()
