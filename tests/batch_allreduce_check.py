"""Child process of tests/test_batch.py: one rank of a data-parallel run.  Every
rank simulates its own share of the batch (its own initial state, so its own
learned weights), then the weights are summed over the batch AND over the ranks
(NCCL all-reduce of the custom update's target) and the global mean is written
back; every rank must end with the same weights, equal to the mean over all
batch elements of all ranks.

    python -m torch.distributed.run --nproc-per-node 2 tests/batch_allreduce_check.py"""
import os
import sys

import numpy as np

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def main():
    import torch
    import torch.distributed as dist
    from tests.test_batch import _model, BATCH
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    model, sg = _model(v_seed=100 + rank)       # same network, another share of the batch
    model.add_custom_update("mean_g", "gradient", "SUM", (sg, "g"), broadcast=True, scale=1.0 / (BATCH * world))
    # a second update of the same group with the other operation: both travel in the one packed buffer
    model.add_custom_update("max_v", "gradient", "MAX", (model.neuron_populations["post"], "V"))
    model.build()
    model.load(device=local)
    rt = model._runtime
    rt.step_time(150)
    g = rt.array("syn.g")
    local_sum = g.sum(axis=0, dtype=np.float64)
    gathered = [None] * world
    dist.all_gather_object(gathered, local_sum)
    want = sum(gathered) / (BATCH * world)
    v_all = [None] * world
    dist.all_gather_object(v_all, rt.array("post.V").max(axis=0))
    rt.init_data_parallel()
    model.custom_update("gradient")
    model.custom_updates["max_v"].vars["reduction"].pull_from_device()
    assert np.array_equal(model.custom_updates["max_v"].vars["reduction"].view, np.max(np.stack(v_all), axis=0))
    after = rt.array("syn.g")
    for b in range(BATCH):
        np.testing.assert_allclose(after[b], want, rtol=1e-5, atol=1e-6)
    rt.close()
    dist.barrier()
    if rank == 0:
        print(f"batch_allreduce_check ok: {world} ranks x {BATCH} batch elements")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
