"""The reference's OWN feature tests (GeNN 5.4.0 tests/features, unmodified) run against the B200 backend,
selected the way a user selects any GeNN backend: GeNNModel(..., backend="b200").

oracle/Makefile.pygenn builds PyGeNN and the `b200_backend` extension module next to it and installs the
reference's test files beside them; genn_b200.pygenn_plugin.register() adds the module to PyGeNN's backend
table.  The tests' `backend` fixture is parametrised over that table, so `-k b200` runs every test on the
plug-in, at batch size 1 and 5.

Every feature file of the reference runs except test_cuda_interface.py (CuPy interop of the CUDA backend's
arrays).  test_custom_connectivity_update.py imports `bitarray`, which this image does not have:
tests/standins/bitarray supplies the few operations it uses (checked against the reference's CPU backend, on
which the file passes with it)."""
import os
import re
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SITE = os.path.join(REPO, "oracle", "_ref", "pygenn_site")
FILES = ["test_event_propagation.py", "test_sparse.py", "test_wu_vars.py", "test_recording.py", "test_custom_update.py",
         "test_pre_post_neuron_vars.py", "test_post_psm_vars.py", "test_event_times.py", "test_continuous_propagation.py",
         "test_egp.py", "test_model_lifecycle.py", "test_model_timing.py", "test_connect_init.py", "test_num.py", "test_rng.py",
         "test_dynamic_param.py", "test_custom_connectivity_update.py"]


@pytest.mark.gpu
def test_reference_feature_suite_passes_on_the_b200_backend():
    if not os.path.isdir(os.path.join(SITE, "pygenn")):
        pytest.skip("PyGeNN has not been built (make -f oracle/Makefile.pygenn)")
    # generated code of an earlier build of the backend must not be reused (GeNN skips generation when the
    # model's hash is unchanged, and the hash does not cover the backend's own sources)
    import glob
    import shutil
    for stale in glob.glob(os.path.join(SITE, "features", "*_CODE")):
        shutil.rmtree(stale, ignore_errors=True)
    res = subprocess.run([sys.executable, os.path.join(REPO, "tests", "pygenn_features_run.py"), "-q", "-x",
                          "-k", "b200", "--timeout", "300"] + FILES,
                         capture_output=True, text=True, timeout=1500)
    tail = res.stdout[-3000:] + res.stderr[-2000:]
    assert res.returncode == 0, tail
    passed = re.search(r"(\d+) passed", res.stdout)
    assert passed and int(passed.group(1)) >= 138, tail
    print(res.stdout[-300:])


def test_plugin_module_sources_are_in_the_tree():
    for f in ("genn_b200/backend/backend.h", "genn_b200/backend/backend.cc", "genn_b200/backend/pygennBackend.cc",
              "genn_b200/pygenn_plugin.py", "include/genn_b200_gen.cuh", "oracle/Makefile.pygenn"):
        assert os.path.exists(os.path.join(REPO, f)), f
