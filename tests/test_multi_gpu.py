"""Sharding by postsynaptic neuron: host logic on CPU (gloo, two processes) and
the in-kernel spike exchange on two GPUs (child processes)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from genn_b200 import abi, workloads
from genn_b200.plan import Plan, shard_bounds
from genn_b200.resolve import resolve

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_partition_every_population():
    for n in (5, 31, 32, 33, 1000, 77169, 617352):
        for world in (1, 2, 4, 8):
            b = shard_bounds(n, world)
            assert b[0] == 0 and b[-1] == n and len(b) == world + 1
            assert all(x <= y for x, y in zip(b, b[1:]))
            assert all(x % 32 == 0 for x in b[:-1])


def test_sharded_synapses_partition_the_unsharded_network():
    full = resolve(workloads.potjans(neuron_scale=0.005, seed=7, host_connectivity=True, background="dc"))
    world = 2
    shards = [resolve(workloads.potjans(neuron_scale=0.005, seed=7, host_connectivity=True, background="dc",
                                        shard=(r, world))) for r in range(world)]
    for s in full.syns:
        def pairs(net):
            q = net.syn(s.name)
            n_pre = net.pop(q.src).n
            ind = q.ind.reshape(n_pre, q.row_stride)
            mask = np.arange(q.row_stride)[None, :] < q.row_length[:, None]
            pre = np.repeat(np.arange(n_pre), q.row_length)
            return np.stack([pre, ind[mask], q.g[mask.reshape(-1)].view(np.uint32), q.d[mask.reshape(-1)]], axis=1)
        whole = pairs(full)
        parts = np.concatenate([pairs(n) for n in shards])
        key = lambda a: a[np.lexsort(a.T[::-1])]
        assert np.array_equal(key(whole), key(parts)), s.name


def test_sharded_plan_lays_out_one_section_per_process():
    from oracle.oracle import NumpyFactory
    world = 2
    plans = [Plan(resolve(workloads.potjans(neuron_scale=0.005, seed=7, host_connectivity=True, background="dc",
                                            shard=(r, world))), NumpyFactory(), 10, shard=(r, world)) for r in range(world)]
    a, b = plans
    for name, arr in a.arrays.items():
        if name.endswith(".spk") or name.endswith(".spk_cnt"):
            other = b.arrays[name]
            # identical offsets in both arenas: a peer pointer is base + the same offset
            assert arr.handle.offset == other.handle.offset and arr.shape == other.shape and arr.shape[0] == world
    for da, db, p in zip(a.neuron_descs, b.neuron_descs, a.net.pops):
        assert da.first_neuron == p.shard_bounds[0] and db.first_neuron == p.shard_bounds[1]
        assert da.num_update + db.num_update == p.n
        assert (db.spk - b.exchange.ptr) - (da.spk - a.exchange.ptr) == p.runtime_slots * p.list_capacity * 4
    for d in a.synapse_descs:
        assert d.src_sections == world and d.src_spk_slot_stride >= 32
    # the delay rings too: a process that owns a spiking neuron may add into its peers' rings, whose
    # address it derives from its own ring's offset in the arena
    rings = [n for n in a.arrays if n.endswith(".den_delay")]
    assert rings
    for name in rings:
        ra, rb = a.arrays[name], b.arrays[name]
        assert ra.handle.offset == rb.handle.offset and ra.shape == rb.shape
        assert a.exchange.ptr <= ra.ptr < a.exchange.ptr + a.exchange.buf.nbytes


def _gloo_worker(rank, world, port, out):
    import torch.distributed as dist
    from genn_b200.runtime import all_gather_bytes
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    got = all_gather_bytes(bytes([rank]) * 64)
    out.put((rank, got))
    dist.destroy_process_group()


def test_handle_exchange_over_gloo_two_processes():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    for rank in range(2):
        assert results[rank] == [bytes([0]) * 64, bytes([1]) * 64]


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("name,schedule", [("potjans_mini_d1", "lag"), ("potjans_mini_d1", "split"),
                                           ("potjans_mini", "emit"), ("potjans_mini", "emit-direct"),
                                           ("potjans_mini", "emit-tiny"), ("potjans_mini", "split"),
                                           ("potjans_mini", "plain")])
def test_sharded_over_gpus_matches_the_unsharded_reference(name, schedule, world):
    """`world` processes, one GPU each: every rank must see exactly the reference's spikes of the
    unsharded network at every step and hold the golden potentials for its slice."""
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + os.getpid() % 200),
           os.path.join(REPO, "tests", "multigpu_check.py"), name, schedule]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=REPO)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("multigpu_check ok") >= 1
    print(res.stdout[-400:])
