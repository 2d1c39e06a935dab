"""Pin the CPU checker (oracle/genn_oracle.c) to the reference.

The fixtures in tests/golden/ were produced by the unmodified reference
(single_threaded_cpu backend) via tests/golden/make_golden.py.  The checker
must reproduce them bit for bit: spike sets, membrane state, postsynaptic
input buffers and learned weights."""
import numpy as np
import pytest

from genn_b200.resolve import resolve
from oracle.oracle import OracleRunner
from tests import helpers
from tests.cases import CASES


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference_golden(name):
    model, steps, dump_every = CASES[name]()
    net = resolve(model)
    runner = OracleRunner(net, steps)
    got = helpers.run_and_collect(runner, net, steps, dump_every)
    want = helpers.load_golden(name)
    helpers.compare(got, want, exact_state=True)
    runner.close()


def test_oracle_counts_synaptic_events():
    model, steps, _ = CASES["ff_sparse"]()
    net = resolve(model)
    runner = OracleRunner(net, steps)
    runner.step(steps)
    gold = helpers.load_golden("ff_sparse")
    rl = net.syn("syn").row_length
    # every presynaptic spike except those of the final step has been propagated
    sp = gold["spikes_pre"]
    expected = int(rl[sp[sp[:, 0] < steps - 1][:, 1]].sum())
    assert runner.synaptic_events == expected
    runner.close()
