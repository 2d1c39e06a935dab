"""Child process of tests/test_multi_gpu.py: one rank of a model sharded by
postsynaptic neuron over several GPUs.

    python -m torch.distributed.run --nproc-per-node 2 tests/multigpu_check.py <case> [lag|emit|emit-direct|emit-tiny|split|plain]

("emit": near synapses between processes travel through the per-CTA queues; "emit-direct": they are reduced
straight into the other process's rings; "emit-tiny": queues of one entry, so that both ways are taken in the
same step.)

Every rank builds the same network restricted to the synapses onto its slice,
steps it with the persistent kernel (spike lists travel between the GPUs inside
the kernel) and checks that (a) the spikes of ALL populations it sees each step
are exactly the reference's golden spikes of the unsharded network and (b) the
membrane potentials of its own slice match the golden ones."""
import os
import sys

import numpy as np

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def main():
    import torch
    import torch.distributed as dist
    from genn_b200.resolve import resolve
    from genn_b200.runtime import Runtime
    from genn_b200 import workloads
    from tests import helpers

    name = sys.argv[1] if len(sys.argv) > 1 else "potjans_mini"
    schedule = sys.argv[2] if len(sys.argv) > 2 else "lag"
    variant = schedule
    schedule = schedule.split("-")[0]
    lag = schedule == "lag"
    kw = dict(min_delay=0.1, extra_delay_slots=1) if name == "potjans_mini_d1" else {}
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")           # bootstrap only: the spikes do not go through it
    assert name in ("potjans_mini", "potjans_mini_d1")
    model = workloads.potjans(neuron_scale=0.005, seed=7, host_connectivity=True, background="dc", record=True,
                              shard=(rank, world), **kw)
    steps, dump_every = 400, 100
    net = resolve(model)
    rt = Runtime(None, steps, device=local, shard=(rank, world), net=net, sharded_emit=(schedule == "emit"))
    rt.set_option("use_lag", 1 if lag else 0)
    rt.set_option("use_split", 0 if schedule == "plain" else 1)
    rt.set_option("use_emit", 1 if schedule == "emit" else 0)
    rt.set_option("use_near_queues", 0 if variant == "emit-direct" else 1)
    rt.set_option("near_queue_words", 2 if variant == "emit-tiny" else 2048)
    want_schedule = (0 if schedule == "plain" else 2 if (lag and name == "potjans_mini_d1")
                     else 1 if schedule == "split" else 3)
    assert rt.schedule == want_schedule, f"rank {rank}: schedule {rt.schedule}, expected {want_schedule}"
    want = helpers.load_golden(name)
    spikes = {p.name: [] for p in net.pops}
    for s in range(steps):
        rt.step_time(1)
        # a peer's lists of this step land when THAT peer finishes the step
        rt.synchronize()
        dist.barrier()
        for p in net.pops:
            spikes[p.name] += [(s, int(i)) for i in rt.current_spikes(p.name)]
        dist.barrier()
        if (s + 1) % dump_every == 0:
            for p in net.pops:
                lo, hi = p.shard_bounds[rank], p.shard_bounds[rank + 1]
                got = rt.array(f"{p.name}.V")[0][lo:hi]
                helpers.assert_close(got, want[f"V_{p.name}_{s + 1}"][lo:hi], f"rank {rank} V {p.name} step {s + 1}",
                                     1e-5, 2e-6)
    for p in net.pops:
        got = helpers.sorted_pairs(spikes[p.name])
        assert np.array_equal(got, want[f"spikes_{p.name}"]), f"rank {rank}: spikes of {p.name} differ"
    # the same again as ONE launch of many steps with recording
    rt2 = Runtime(None, steps, device=local, shard=(rank, world), net=resolve(
        workloads.potjans(neuron_scale=0.005, seed=7, host_connectivity=True, background="dc", record=True,
                          shard=(rank, world), **kw)), sharded_emit=(schedule == "emit"))
    rt2.set_option("use_lag", 1 if lag else 0)
    rt2.set_option("use_split", 0 if schedule == "plain" else 1)
    rt2.set_option("use_emit", 1 if schedule == "emit" else 0)
    rt2.set_option("use_near_queues", 0 if variant == "emit-direct" else 1)
    rt2.set_option("near_queue_words", 2 if variant == "emit-tiny" else 2048)
    dist.barrier()
    rt2.step_time(steps)
    rt2.synchronize()
    rt2.pull_recording_buffers()
    for p in rt2.net.pops:
        times, ids = rt2.recorded_spikes(p.name)[0]
        lo, hi = p.shard_bounds[rank], p.shard_bounds[rank + 1]
        got = helpers.sorted_pairs(np.stack([np.rint(times / net.dt).astype(np.uint32), ids], axis=1))
        ref = want[f"spikes_{p.name}"]
        ref = ref[(ref[:, 1] >= lo) & (ref[:, 1] < hi)]
        assert np.array_equal(got, ref), f"rank {rank}: recorded spikes of {p.name} differ"
    dist.barrier()
    rt.close()
    rt2.close()
    if rank == 0:
        print(f"multigpu_check ok: {name} {variant}, {world} ranks, schedule {want_schedule}, "
              f"{sum(len(v) for v in spikes.values())} spikes")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
