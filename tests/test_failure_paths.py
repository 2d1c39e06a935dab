"""Failure detection without faulting anything: every wait inside the persistent kernels is bounded, a wait
that runs out sets an error bit, all CTAs leave the kernel and the host reports B200_ERR_DEVICE_CHECK; the CUDA
context stays usable.

The failure is made on the host side of the protocol: a runner is configured as rank 0 of a two-process model
whose "peer" is a zeroed buffer in the same process, so the count words rank 1 would write never arrive.  The
wait limit is set to a few thousand polls (well under a millisecond).  No kernel traps, no address is bad, no
loop is unbounded."""
import numpy as np
import pytest

from genn_b200 import abi, workloads
from genn_b200.resolve import resolve

pytestmark = pytest.mark.gpu


def _net(shard=None):
    return resolve(workloads.potjans(neuron_scale=0.005, seed=7, host_connectivity=True, background="dc", record=True,
                                     shard=shard))


def test_missing_peer_runs_into_the_wait_limit_and_the_gpu_stays_usable():
    import torch
    from genn_b200.runtime import Runtime
    keep = []

    def silent_peer(nbytes):
        keep.append(torch.zeros(nbytes, dtype=torch.uint8, device="cuda"))
        return keep[-1].data_ptr()

    rt = Runtime(None, 10, net=_net(shard=(0, 2)), shard=(0, 2), local_peers={1: silent_peer},
                 exchange=lambda mine: [mine, mine])
    rt.set_option("exchange_spin_limit", 4000)
    rt.set_option("barrier_spin_limit", 200000)
    rt.step_time(3)
    with pytest.raises(abi.B200Error, match="did not arrive in time"):
        rt.synchronize()
    rt.close()

    # the same GPU, the same process: an unsharded runner steps and matches its golden potentials
    from tests import helpers
    net = _net()
    ok = Runtime(None, 400, net=net)
    ok.step_time(400)
    ok.synchronize()
    want = helpers.load_golden("potjans_mini")
    for p in net.pops:
        helpers.assert_close(ok.array(f"{p.name}.V")[0], want[f"V_{p.name}_400"], f"V {p.name}", 1e-5, 2e-6)
    ok.close()


def test_wait_limits_are_options():
    from genn_b200.runtime import Runtime
    rt = Runtime(None, 10, net=_net())
    for name in ("barrier_spin_limit", "exchange_spin_limit", "stream_wait_cycles"):
        rt.set_option(name, 12345)
        with pytest.raises(abi.B200Error):
            rt.set_option(name, 0)
    rt.close()
