"""The B200 code-generation backend as a GeNN plug-in.

`oracle/_ref/b200_driver` is the reference driver (oracle/ref_driver.cc) compiled with the B200 backend
(genn_b200/backend) selected instead of GeNN's single_threaded_cpu backend: the model goes through GeNN's own
ModelSpec, group merging, transpiler, generateAll and Runtime, unmodified; only the backend behind
GeNN::CodeGenerator::BackendBase differs.

Without a GPU: the generated code of a network with NON-built-in neuron and weight update models compiles
for sm_100a and contains the models' arithmetic inlined into the backend's kernel scaffolds.
With a GPU: the same networks the CUDA library is pinned with (tests/golden, produced by the reference's CPU
backend) and the custom-model network run through the plug-in; spikes must be identical, state within 1e-5."""
import glob
import os
import shutil
import subprocess
import tempfile

import numpy as np
import pytest

from genn_b200.resolve import resolve, write_netspec
from tests import helpers, plugin_cases
from tests.cases import CASES

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
B200_DRIVER = os.path.join(REPO, "oracle", "_ref", "b200_driver")
CPU_DRIVER = os.path.join(REPO, "oracle", "_ref", "ref_driver")
RTOL, ATOL = 1e-5, 2e-6


def _need(path):
    if not os.path.exists(path):
        pytest.skip(f"{path} has not been built (python -c 'import __graft_entry__ as g; g.build()')")


def _run(driver, spec, work, out, *extra):
    os.makedirs(out, exist_ok=True)
    os.makedirs(work, exist_ok=True)
    res = subprocess.run([driver, spec, os.path.join(work, "build"), out, *extra], capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res


def _collect(out):
    data = {}
    for path in glob.glob(os.path.join(out, "*.bin")):
        name = os.path.basename(path)[:-4]
        if name.startswith("spikes_"):
            data[name] = helpers.sorted_pairs(np.fromfile(path, dtype=np.uint32))
        elif not name.startswith("denDelay_"):
            data[name] = np.fromfile(path, dtype=np.float32)
    return data


@pytest.fixture
def workdir():
    d = tempfile.mkdtemp(prefix="plugin_")
    yield d
    shutil.rmtree(d, ignore_errors=True)


def test_generated_code_for_custom_models_compiles_for_sm100a(workdir):
    """No GPU needed: GeNN generates through the B200 backend and nvcc compiles the result."""
    _need(B200_DRIVER)
    spec = plugin_cases.custom_models(os.path.join(workdir, "spec"))
    _run(B200_DRIVER, spec, workdir, os.path.join(workdir, "out"), "generate")
    code = os.path.join(workdir, "build", "custom_models_CODE")
    assert os.path.exists(os.path.join(code, "librunner.so"))
    neuron = open(os.path.join(code, "neuronUpdate.cc")).read()
    synapse = open(os.path.join(code, "synapseUpdate.cc")).read()
    makefile = open(os.path.join(code, "Makefile")).read()
    # the custom sim code and the custom weight update code, transpiled and inlined
    assert "_drive" in neuron and "b200gen::emitEvents" in neuron and "__global__" in neuron
    assert "gScale" in synapse and "fmin(" in synapse and "atomicAdd(&group->outPost" in synapse
    assert "compute_100a,code=sm_100a" in makefile
    # the symbols GeNN's runtime looks up (runtime.cc:81-119)
    symbols = subprocess.check_output(["nm", "-D", "--defined-only", os.path.join(code, "librunner.so")], text=True)
    for name in ("allocateMem", "freeMem", "initialize", "initializeSparse", "stepTime", "updateNeurons", "updateSynapses",
                 "pushMergedNeuronUpdateGroup0ToDevice", "pushMergedPresynapticUpdateGroup0ToDevice", "neuronUpdateTime"):
        assert f" {name}\n" in symbols, f"{name} not exported by the generated library"


@pytest.mark.gpu
def test_custom_models_match_the_reference_cpu_backend(workdir):
    """A neuron model and a weight update model GeNN does not ship: same spec through GeNN + CPU backend and
    through GeNN + B200 backend."""
    _need(B200_DRIVER)
    _need(CPU_DRIVER)
    spec = plugin_cases.custom_models(os.path.join(workdir, "spec"))
    _run(CPU_DRIVER, spec, os.path.join(workdir, "cpu"), os.path.join(workdir, "out_cpu"))
    _run(B200_DRIVER, spec, os.path.join(workdir, "b200"), os.path.join(workdir, "out_b200"))
    want, got = _collect(os.path.join(workdir, "out_cpu")), _collect(os.path.join(workdir, "out_b200"))
    assert len(want["spikes_q"]) > 1000, "the network was meant to fire"
    # spikes exactly; state within 1e-5 where the quadratic neuron contracts (below its critical potential of
    # -40 mV).  On its upswing towards a spike the model multiplies any difference in its summed input (fp32
    # sums into a shared target are unordered on a GPU) by e every few hundred microseconds: 2e-3 there.
    for key, w in want.items():
        g = got[key]
        if key.startswith("spikes_"):
            assert np.array_equal(g, w), f"{key}: spike sets differ ({len(g)} vs {len(w)} spikes)"
        elif key.startswith("V_q"):
            rising = w >= -40.0
            helpers.assert_close(g[~rising], w[~rising], key + " (contracting)", RTOL, ATOL)
            helpers.assert_close(g[rising], w[rising], key + " (upswing)", 2e-3, 1e-3)
        else:
            helpers.assert_close(g, w, key, RTOL, ATOL)


@pytest.mark.gpu
@pytest.mark.parametrize("name", [n for n in CASES if n != "c1_full"] + ["c1_full"])
def test_golden_networks_through_the_plugin(name, workdir):
    """The networks of tests/golden (reference CPU backend) through GeNN's runtime on the B200 backend: built-in
    LIF / Izhikevich / SpikeSourceArray, ExpCurr / ExpCond / DeltaCurr, StaticPulse(+ConstantWeight, +DendriticDelay),
    STDP with postsynaptic learning over the remap, SPARSE / BITMASK / DENSE, axonal and dendritic delays."""
    _need(B200_DRIVER)
    model, steps, dump_every = CASES[name]()
    spec = write_netspec(resolve(model), os.path.join(workdir, "spec"), steps, dump_every)
    _run(B200_DRIVER, spec, workdir, os.path.join(workdir, "out"))
    helpers.compare(_collect(os.path.join(workdir, "out")), helpers.load_golden(name), exact_state=False, rtol=RTOL, atol=ATOL)


@pytest.mark.gpu
def test_potjans_through_the_plugin_fires_like_the_library(workdir, capsys):
    """The Potjans architecture at a tenth of its neurons (published in-degrees: 30 M synapses, dendritic delays,
    constant-current background) through GeNN's runtime on the B200 backend: per-population rates over 0.2 s must
    agree with the descriptor library's run of the same arrays (a chaotic network: 10 %), and the time per step of
    GeNN's stepTime loop is printed (one launch per kernel, as GeNN's runtime drives it)."""
    from genn_b200 import workloads
    from genn_b200.runtime import Runtime
    _need(B200_DRIVER)
    steps = 2000
    model = workloads.potjans(neuron_scale=0.1, seed=99, host_connectivity=True, background="dc", record=True)
    net = resolve(model)
    spec = write_netspec(net, os.path.join(workdir, "spec"), steps, 0)
    with open(spec, "a") as f:
        f.write("timing 0\n")          # GeNN's per-kernel timers synchronise after every kernel group
    _run(B200_DRIVER, spec, workdir, os.path.join(workdir, "out"))
    timing = dict(l.split() for l in open(os.path.join(workdir, "out", "timing.txt")))
    got = _collect(os.path.join(workdir, "out"))
    rt = Runtime(None, steps, net=net)
    rt.step_time(steps)
    rt.synchronize()
    rt.pull_recording_buffers()
    total = 0
    for p in net.pops:
        lib = len(rt.recorded_spikes(p.name)[0][1]) / p.n
        plug = len(got[f"spikes_{p.name}"]) / p.n
        total += len(got[f"spikes_{p.name}"])
        assert abs(plug - lib) <= 0.1 * max(lib, plug) + 0.02, f"{p.name}: {plug:.3f} spikes per neuron through the plug-in, {lib:.3f} in the library"
    rt.close()
    assert total > 1000
    with capsys.disabled():
        print(f"\nplug-in: Potjans x0.1, {steps} steps, {float(timing['loop_seconds']) / steps * 1e6:.1f} us per step "
              f"in GeNN's stepTime loop, {total} spikes")
