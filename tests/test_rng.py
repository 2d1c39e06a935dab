"""The library's random streams (include/genn_b200_rng.h), checked on the CPU
through the checker build: Philox known answers, distribution moments and the
PoissonExp current source against its analytic mean."""
import ctypes
import os
import subprocess
import tempfile

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r'''
#include <stdio.h>
#include "genn_b200_rng.h"
int main(void) {
    /* Philox4x32-10 known-answer vectors published with the algorithm (Random123 kat_vectors) */
    b200_philox_out o = b200_philox4x32_10(0, 0, 0, 0, 0, 0);
    printf("%08x %08x %08x %08x\n", o.x[0], o.x[1], o.x[2], o.x[3]);
    o = b200_philox4x32_10(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
    printf("%08x %08x %08x %08x\n", o.x[0], o.x[1], o.x[2], o.x[3]);
    o = b200_philox4x32_10(0x243f6a88u, 0x85a308d3u, 0x13198a2eu, 0x03707344u, 0xa4093822u, 0x299f31d0u);
    printf("%08x %08x %08x %08x\n", o.x[0], o.x[1], o.x[2], o.x[3]);
    /* moments */
    double su = 0, su2 = 0, sn = 0, sn2 = 0, sp = 0, sp2 = 0;
    const int N = 400000;
    const float lambda = 1.6f, eml = expf(-1.6f);
    for(int i = 0; i < N; i++) {
        b200_rng r = b200_rng_init(42, 3, (uint64_t)i);
        const float u = b200_rng_uniform(&r);
        const float z = b200_rng_normal(&r);
        su += u; su2 += (double)u * u; sn += z; sn2 += (double)z * z;
        const b200_philox_out blk = b200_rng_step_block(42, 5, (uint32_t)(i / 16), (uint64_t)(i % 16));
        const double k = b200_poisson_inverse(b200_u32_to_uniform(b200_rng_step_word(&blk, (uint64_t)(i % 16))), eml, lambda);
        sp += k; sp2 += k * k;
    }
    printf("%.6f %.6f %.6f %.6f %.6f %.6f\n", su / N, su2 / N - (su / N) * (su / N), sn / N,
           sn2 / N - (sn / N) * (sn / N), sp / N, sp2 / N - (sp / N) * (sp / N));
    /* accuracy of the deterministic elementary functions */
    double el = 0, ee = 0;
    for(int i = 1; i < 100000; i++) {
        const float u = i / 100000.0f, x = -80.0f * i / 100000.0f;
        const double a = fabs(b200_logf(u) - log((double)u)) / (fabs(log((double)u)) + 1e-3);
        const double b = fabs(b200_expf(x) - exp((double)x)) / exp((double)x);
        if(a > el) el = a;
        if(b > ee) ee = b;
    }
    printf("%.3e %.3e\n", el, ee);
    return 0;
}
'''


@pytest.fixture(scope="module")
def output():
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "t.c")
        open(c, "w").write(SRC)
        exe = os.path.join(d, "t")
        subprocess.check_call(["/usr/bin/gcc", "-O2", "-ffp-contract=off", "-I", os.path.join(REPO, "include"),
                               c, "-o", exe, "-lm"])
        return subprocess.check_output([exe]).decode().splitlines()


def test_philox_known_answers(output):
    assert output[0] == "6627e8d5 e169c58d bc57ac4c 9b00dbd8"
    assert output[1] == "408f276d 41c83b0e a20bc7c6 6d5451fd"
    assert output[2] == "d16cfe09 94fdcceb 5001e420 24126ea1"


def test_distribution_moments(output):
    mu, vu, mn, vn, mp, vp = (float(x) for x in output[3].split())
    assert abs(mu - 0.5) < 2e-3 and abs(vu - 1.0 / 12.0) < 1e-3
    assert abs(mn) < 5e-3 and abs(vn - 1.0) < 1e-2
    assert abs(mp - 1.6) < 1e-2 and abs(vp - 1.6) < 2e-2      # Poisson: mean = variance = lambda


def test_elementary_functions_accuracy(output):
    el, ee = (float(x) for x in output[4].split())
    assert el < 1e-6 and ee < 1e-6


def test_poisson_exp_mean_current_matches_analytic():
    """A PoissonExp source into a passive LIF neuron: the mean injected current
    is weight * tauSyn * rate (currentSourceModels.h:107-129)."""
    from genn_b200 import GeNNModel
    from genn_b200.resolve import resolve
    from oracle.oracle import OracleRunner
    m = GeNNModel("float", "pe")
    m.dt = 0.1
    m.seed = 5
    lif = {"C": 0.25, "TauM": 10.0, "Vrest": -65.0, "Vreset": -65.0, "Vthresh": 1000.0, "Ioffset": 0.0, "TauRefrac": 2.0}
    pop = m.add_neuron_population("p", 2000, "LIF", lif, {"V": -65.0, "RefracTime": 0.0})
    m.add_current_source("cs", "PoissonExp", pop, {"weight": 0.0878, "tauSyn": 0.5, "rate": 16000.0}, {"current": 0.0})
    r = OracleRunner(resolve(m), None)
    r.step(500)
    # in the steady state V = Vrest + R * mean(I), R = TauM / C
    mean_i = 0.0878 * 0.5 * 16.0
    v = r.array("p.V")[0].mean()
    assert abs((v + 65.0) / (mean_i * 40.0) - 1.0) < 0.02
    r.close()
