"""Batched simulation (batch size > 1: every kernel's batch dimension) and the
batch-reduce custom update (backendSIMT.cc:888-927, 1109-1147), against the CPU
checker; the host side of a data-parallel reduction on CPU (gloo) and, with two
GPUs, the reduction itself (one packed NCCL all-reduce inside b200_custom_update)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from genn_b200 import GeNNModel, init_postsynaptic, init_weight_update
from genn_b200.resolve import resolve
from genn_b200 import workloads
from tests import helpers

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BATCH, STEPS = 3, 200


def _model(seed=9, batch=BATCH, v_seed=77):
    """Spike sources -> LIF through SPARSE connectivity with additive STDP; every batch element
    starts from its own membrane potentials, so the elements diverge and so do their weights."""
    rng = np.random.default_rng(seed)
    m = GeNNModel("float", "batched")
    m.dt = 1.0
    m.batch_size = batch
    npre, npost = 120, 60
    start, end, times = workloads.poisson_spike_trains(rng, npre, 40.0, STEPS * m.dt)
    src = m.add_neuron_population("pre", npre, "SpikeSourceArray", {}, {"startSpike": start, "endSpike": end})
    src.set_extra_global_param("spikeTimes", times)
    lif = {"C": 1.0, "TauM": 20.0, "Vrest": -65.0, "Vreset": -70.0, "Vthresh": -55.0, "Ioffset": 0.0, "TauRefrac": 2.0}
    v0 = np.random.default_rng(v_seed).uniform(-70.0, -56.0, size=(batch, npost)).astype(np.float32)
    trg = m.add_neuron_population("post", npost, "LIF", lif, {"V": v0, "RefracTime": 0.0})
    trg.spike_recording_enabled = True
    mask = rng.random((npre, npost)) < 0.4
    pre, post = np.nonzero(mask)
    g = rng.uniform(0.0, 0.5, size=len(pre)).astype(np.float32)
    sg = m.add_synapse_population("syn", "SPARSE", src, trg,
                                  init_weight_update("STDP", {"tauPlus": 20.0, "tauMinus": 20.0, "Aplus": 0.01,
                                                              "Aminus": 0.0105, "Wmin": 0.0, "Wmax": 1.0}, {"g": g}),
                                  init_postsynaptic("ExpCurr", {"tau": 5.0}))
    sg.set_sparse_connections(pre, post)
    return m, sg


def _static_batched(batch=2):
    """Potjans miniature (dendritic delays, constant-current background) with a different initial
    potential for every batch element."""
    m = workloads.potjans(neuron_scale=0.005, seed=7, host_connectivity=True, background="dc", record=True)
    m.batch_size = batch
    net = resolve(m)
    rng = np.random.default_rng(21)
    for p in net.pops:
        p.vars["V"] = (p.vars["V"] + rng.normal(0.0, 2.0, size=p.vars["V"].shape)).astype(np.float32)
    return net


@pytest.mark.gpu
@pytest.mark.parametrize("tiled", [0, 1])
def test_batched_static_network_matches_the_cpu_checker(tiled):
    """Batch > 1 through the SPARSE kernels of the one-launch-per-kernel path: one reduction per event
    (tiled 0) and the target-tiled kernel forced on for every step (tiled 1)."""
    from genn_b200.runtime import Runtime
    from oracle.oracle import OracleRunner
    net, onet = _static_batched(), _static_batched()
    rt, orc = Runtime(None, 300, net=net), OracleRunner(onet, 300)
    rt.set_option("tiled_min_events", 0 if tiled else 1e30)
    different = False
    for step in range(300):
        rt.step_time(1)
        orc.step(1)
        for p in net.pops:
            a, b = np.sort(rt.current_spikes(p.name, 0)), np.sort(rt.current_spikes(p.name, 1))
            different = different or not np.array_equal(a, b)
            for e, got in enumerate((a, b)):
                assert np.array_equal(got, np.sort(orc.current_spikes(p.name, e))), f"step {step} {p.name}[{e}]"
    for p in net.pops:
        helpers.assert_close(rt.array(f"{p.name}.V").reshape(-1), orc.array(f"{p.name}.V").reshape(-1), f"V {p.name}", 1e-5, 2e-6)
    assert different, "the batch elements were meant to diverge"
    assert rt.counter("heavy") == tiled
    rt.close()
    orc.close()


@pytest.mark.gpu
def test_every_batch_element_matches_the_cpu_checker_and_the_weights_reduce():
    from genn_b200.runtime import Runtime
    from oracle.oracle import OracleRunner
    model, sg = _model()
    model.add_custom_update("mean_g", "gradient", "SUM", (sg, "g"), broadcast=True, scale=1.0 / BATCH)
    model.add_custom_update("max_v", "gradient", "MAX", (model.neuron_populations["post"], "V"))
    model.build()
    model.load(num_recording_timesteps=STEPS)
    rt = model._runtime
    net = rt.net
    orc = OracleRunner(resolve(_model()[0]), STEPS)
    diverged = False
    for step in range(STEPS):
        rt.step_time(1)
        orc.step(1)
        for b in range(BATCH):
            assert np.array_equal(np.sort(rt.current_spikes("post", b)), np.sort(orc.current_spikes("post", b))), \
                f"step {step} batch {b}: spikes differ"
        if step % 40 == 39:
            for name in ("post.V", "psm0.out_post", "syn.g"):
                helpers.assert_close(rt.array(name), orc.array(name), f"step {step} {name}", 1e-5, 2e-6)
            g = rt.array("syn.g")
            diverged = diverged or not np.array_equal(g[0], g[1])
    assert diverged, "the batch elements were meant to learn different weights"
    # batch reduction: sum of the weights over the batch, mean written back; maximum of V
    g_before, v_before, orc_v_before = rt.array("syn.g"), rt.array("post.V"), orc.array("post.V")
    model.custom_update("gradient")
    orc_sum = orc.add_custom_update("SUM", "syn.g", True, 1.0 / BATCH)
    orc_max = orc.add_custom_update("MAX", "post.V")
    orc.custom_update()
    model.custom_updates["mean_g"].vars["reduction"].pull_from_device()
    model.custom_updates["max_v"].vars["reduction"].pull_from_device()
    got_sum = model.custom_updates["mean_g"].vars["reduction"].view
    want_sum = g_before[0] + g_before[1] + g_before[2]         # the kernel adds in batch order
    assert np.array_equal(got_sum, want_sum.reshape(-1))
    helpers.assert_close(got_sum, orc.array(orc_sum), "reduced weights vs checker", 1e-6, 1e-7)
    assert np.array_equal(model.custom_updates["max_v"].vars["reduction"].view, v_before.max(axis=0))
    assert np.array_equal(orc.array(orc_max), orc_v_before.max(axis=0))
    g_after = rt.array("syn.g")
    for b in range(BATCH):
        assert np.array_equal(g_after[b], (want_sum * np.float32(1.0 / BATCH)).reshape(g_after[b].shape))
    helpers.assert_close(g_after, orc.array("syn.g"), "weights after the broadcast vs checker", 1e-6, 1e-7)
    # and the run goes on from the averaged weights
    rt.step_time(20)
    orc.step(20)
    helpers.assert_close(rt.array("post.V"), orc.array("post.V"), "V after the update", 1e-5, 2e-6)
    model.unload() if hasattr(model, "unload") else rt.close()
    orc.close()


def _gloo_worker(rank, world, port, out):
    """The host side of init_data_parallel: rank 0's 128-byte id reaches every rank."""
    import torch.distributed as dist
    from genn_b200.runtime import all_gather_bytes
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ident = (bytes(range(128)) if rank == 0 else bytes(128))
    everyone = all_gather_bytes(ident)
    out.put((rank, len(everyone), everyone[0]))
    dist.destroy_process_group()


def test_communicator_id_reaches_both_processes_over_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29400 + os.getpid() % 90
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    for _, n, first in results:
        assert n == 2 and first == bytes(range(128))


@pytest.mark.gpu
def test_data_parallel_reduction_over_nccl_on_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(29900 + os.getpid() % 90), os.path.join(REPO, "tests", "batch_allreduce_check.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=REPO)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "batch_allreduce_check ok" in res.stdout


@pytest.mark.gpu
def test_bench_workloads_build_and_step_at_small_size():
    """The C4 and C5 workloads of bench.py at a size that runs in a second: PROCEDURAL stress network with 32 threads
    per spike, batched STDP with its batch-reduce custom update."""
    m = workloads.procedural_stress(num_neurons=4000, prob=0.01, threads_per_spike=32, record=True)
    m.build()
    m.load(num_recording_timesteps=50)
    rt = m._runtime
    rt.set_option("count_events", 1)
    m.step_time(50)
    rt.synchronize()
    assert rt.counter("spikes") > 0 and rt.counter("synaptic_events") > 0
    m.unload()

    m, sg = workloads.batched_stdp(num_pre=300, num_post=200, batch=4)
    m.build()
    m.load()
    rt = m._runtime
    m.step_time(100)
    g = rt.array("syn.g")
    m.custom_update("gradient")
    after = rt.array("syn.g")
    want = g.sum(axis=0, dtype=np.float64) / 4
    for b in range(4):
        np.testing.assert_allclose(after[b], want, rtol=1e-5, atol=1e-6)
    m.unload()
