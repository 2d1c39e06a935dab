"""Regenerate tests/golden/stats_*.json: per-population firing rate and CV-ISI
of the config-scale networks of tests/cases.py (STATS_CASES) over 10 s of
simulated time, produced by the UNMODIFIED reference (GeNN 5.4.0
single_threaded_cpu backend) loaded with the host-generated connectivity.

    make -f oracle/Makefile.ref -j8
    python tests/golden/make_stats_golden.py potjans_x1 cond_ei

Only the 2 x (number of populations) statistics are committed; the spec files
(a few GB) and spike lists live in a temporary directory."""
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)

from genn_b200 import stats                            # noqa: E402
from genn_b200.resolve import resolve, write_netspec   # noqa: E402
from tests.cases import STATS_CASES                    # noqa: E402


def main():
    for name in sys.argv[1:] or list(STATS_CASES):
        model, steps = STATS_CASES[name]()
        net = resolve(model)
        work = tempfile.mkdtemp(prefix="stats_golden_", dir=os.environ.get("TMPDIR", "/tmp"))
        try:
            spec = write_netspec(net, os.path.join(work, "spec"), steps, 0)
            out = os.path.join(work, "out")
            os.makedirs(out)
            t0 = time.time()
            subprocess.check_call([os.path.join(REPO, "oracle", "_ref", "ref_driver"), spec,
                                   os.path.join(work, "work"), out])
            wall = time.time() - t0
            timing = dict(l.split() for l in open(os.path.join(out, "timing.txt")))
            pops = {}
            for p in net.pops:
                sp = np.fromfile(os.path.join(out, f"spikes_{p.name}.bin"), dtype=np.uint32).reshape(-1, 2)
                pops[p.name] = stats.rate_and_cv(sp[:, 0], sp[:, 1], p.n, steps * net.dt * 1e-3)
        finally:
            shutil.rmtree(work, ignore_errors=True)
        doc = {"case": name, "seed": int(model.seed), "steps": steps, "dt_ms": net.dt,
               "neurons": int(sum(p.n for p in net.pops)),
               "synapses": int(sum(int(s.row_length.sum()) for s in net.syns)),
               "produced_by": "GeNN 5.4.0 single_threaded_cpu backend (oracle/_ref/ref_driver), g++ -O3",
               "reference_loop_seconds": float(timing["loop_seconds"]), "wall_seconds": wall,
               "populations": pops}
        with open(os.path.join(HERE, f"stats_{name}.json"), "w") as f:
            json.dump(doc, f, indent=1)
        print(name, json.dumps(pops))


if __name__ == "__main__":
    main()
