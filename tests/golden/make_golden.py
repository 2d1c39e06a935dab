"""Regenerate tests/golden/*.npz by running the UNMODIFIED reference
(GeNN 5.4.0 single_threaded_cpu backend) on the networks of tests/cases.py.

    make -f oracle/Makefile.ref -j8 [REF=<reference tree>]   # builds oracle/_ref/
    python tests/golden/make_golden.py

Each fixture holds the per-step spike (step, id) pairs of every population and
the membrane potentials, postsynaptic input buffers and (for learning rules)
weights at the dump steps, exactly as the reference produced them."""
import glob
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)

from genn_b200.resolve import resolve, write_netspec   # noqa: E402
from tests.cases import CASES                          # noqa: E402


def run_reference(net, steps, dump_every, workdir):
    spec = write_netspec(net, os.path.join(workdir, "spec"), steps, dump_every)
    out = os.path.join(workdir, "out")
    os.makedirs(out, exist_ok=True)
    driver = os.path.join(REPO, "oracle", "_ref", "ref_driver")
    subprocess.check_call([driver, spec, os.path.join(workdir, "work"), out])
    data = {}
    for path in glob.glob(os.path.join(out, "*.bin")):
        name = os.path.basename(path)[:-4]
        if name.startswith("spikes_"):
            sp = np.fromfile(path, dtype=np.uint32).reshape(-1, 2)
            data[name] = sp[np.lexsort((sp[:, 1], sp[:, 0]))]
        elif name.startswith("denDelay_"):
            continue
        else:
            data[name] = np.fromfile(path, dtype=np.float32)
    return data


def main():
    names = sys.argv[1:] or list(CASES)
    for name in names:
        model, steps, dump_every = CASES[name]()
        net = resolve(model)
        work = tempfile.mkdtemp(prefix="golden_")
        try:
            data = run_reference(net, steps, dump_every, work)
        finally:
            shutil.rmtree(work, ignore_errors=True)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **data)
        print(name, {k: v.shape for k, v in sorted(data.items())})


if __name__ == "__main__":
    main()
