"""Recurrent networks at benchmark size against the reference's CPU backend.

A recurrent spiking network is chaotic: two correct simulators part company
spike by spike within a few hundred steps (fp32 sums into a shared target are
unordered on a GPU), so config-scale parity is statistical.  The reference
(GeNN 5.4.0 single_threaded_cpu backend, unmodified) was run for 10 s of
simulated time on the host-generated networks of tests/cases.py
(STATS_CASES) by tests/golden/make_stats_golden.py; only its per-population
firing rates and CV-ISI are committed.  Here the CUDA path simulates the same
arrays for the same 10 s; both statistics must agree within 2 %."""
import json
import os

import numpy as np
import pytest

from genn_b200 import stats
from tests import helpers
from tests.cases import STATS_CASES

TOLERANCE = 0.02
BLOCK = 10000


def _golden(name):
    path = os.path.join(helpers.GOLDEN, f"stats_{name}.json")
    if not os.path.exists(path):
        pytest.skip(f"{path} has not been generated")
    return json.load(open(path))


def simulate_statistics(model, steps, block=BLOCK, device=0):
    """Run `steps` time steps in blocks, decoding the spike recording of each block; returns
    {population: rate_and_cv}."""
    model.build()
    model.load(num_recording_timesteps=block, device=device)
    rt = model._runtime
    net = rt.net
    spikes = {p.name: ([], []) for p in net.pops}
    done = 0
    while done < steps:
        n = min(block, steps - done)
        assert n == block, "the step count must be a multiple of the block length"
        model.step_time(n)
        model.pull_recording_buffers_from_device()
        for p in net.pops:
            times, ids = rt.recorded_spikes(p.name)[0]
            spikes[p.name][0].append(np.rint(times / net.dt).astype(np.int64))
            spikes[p.name][1].append(ids)
        done += n
    out = {p.name: stats.rate_and_cv(np.concatenate(spikes[p.name][0]), np.concatenate(spikes[p.name][1]), p.n,
                                     steps * net.dt * 1e-3) for p in net.pops}
    model.unload()
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(STATS_CASES))
def test_rates_and_cv_isi_within_two_percent_of_the_reference(name):
    golden = _golden(name)
    model, steps = STATS_CASES[name]()
    assert steps == golden["steps"]
    got = simulate_statistics(model, steps)
    rate_err, cv_err = stats.compare(got, golden["populations"])
    report = {p: (round(got[p]["rate_hz"], 4), round(golden["populations"][p]["rate_hz"], 4),
                  round(got[p]["cv_isi"], 4), round(golden["populations"][p]["cv_isi"], 4)) for p in got}
    assert rate_err <= TOLERANCE and cv_err <= TOLERANCE, \
        f"{name}: rate error {rate_err:.4f}, CV-ISI error {cv_err:.4f}; (rate, ref rate, cv, ref cv) = {report}"


def test_statistics_helper_on_known_trains():
    # neuron 0: perfectly regular (CV 0); neuron 1: intervals 1, 3, 1, 3 (mean 2, sd 1 -> CV 0.5); neuron 2 silent
    steps = np.array([0, 10, 20, 30, 0, 1, 4, 5, 8])
    ids = np.array([0, 0, 0, 0, 1, 1, 1, 1, 1])
    r = stats.rate_and_cv(steps, ids, 3, 1.0)
    assert r["rate_hz"] == pytest.approx(3.0)
    assert r["neurons_in_cv"] == 2
    assert r["cv_isi"] == pytest.approx(0.25)
    merged = stats.merge([stats.partial(steps[:4], ids[:4], 1, first_id=0),
                          stats.partial(steps[4:], ids[4:], 2, first_id=1)], 1.0)
    assert merged["rate_hz"] == pytest.approx(3.0) and merged["cv_isi"] == pytest.approx(0.25)


def test_host_drawn_potjans_is_the_same_network_every_time_and_shards_partition_it():
    """The projections are drawn side by side by a thread pool, each from a stream of its own: the result must not
    depend on the scheduling, and the shards of a sharded build must be exactly the unsharded network's synapses."""
    from genn_b200 import workloads
    from genn_b200.resolve import resolve
    a = resolve(workloads.potjans(neuron_scale=0.01, seed=5, host_connectivity=True, background="dc"))
    b = resolve(workloads.potjans(neuron_scale=0.01, seed=5, host_connectivity=True, background="dc"))
    shards = [resolve(workloads.potjans(neuron_scale=0.01, seed=5, host_connectivity=True, background="dc", shard=(r, 2)))
              for r in range(2)]
    total = 0
    for sa, sb in zip(a.syns, b.syns):
        assert np.array_equal(sa.row_length, sb.row_length) and np.array_equal(sa.ind, sb.ind)
        assert np.array_equal(sa.g, sb.g) and np.array_equal(sa.d, sb.d)
        assert int(sa.row_length.sum()) == sum(int(s.syn(sa.name).row_length.sum()) for s in shards)
        total += int(sa.row_length.sum())
    assert total > 100000
