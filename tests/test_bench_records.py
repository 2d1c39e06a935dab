"""bench.py's tracked inputs: the ncu record of the persistent kernel's DRAM traffic must belong to the kernel
sources in the tree (bench.py prints `"traffic": null` otherwise), the reference statistics it compares with must be
complete, and its command line must parse."""
import json
import os
import subprocess
import sys

import numpy as np

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def test_dram_traffic_record_was_taken_on_the_sources_in_the_tree():
    import bench
    per_step, note = bench.captured_traffic("streamStepKernel")
    assert per_step is not None, note + ": re-take the capture described in profiles/dram_traffic.txt"
    # 0.68 MB of algorithmic bytes per step; the capture lies between 1x and 3x of that
    assert 0.6e6 < per_step < 2.1e6


def test_reference_statistics_cover_every_population():
    for name, pops in (("stats_potjans_x1.json", ["23E", "23I", "4E", "4I", "5E", "5I", "6E", "6I"]), ("stats_cond_ei.json", ["E", "I"])):
        doc = json.load(open(os.path.join(REPO, "tests", "golden", name)))
        assert doc["steps"] == 100000 and "single_threaded_cpu" in doc["produced_by"]
        for p in pops:
            assert doc["populations"][p]["rate_hz"] > 0.5 and 0.5 < doc["populations"][p]["cv_isi"] < 1.5


def test_bench_command_line():
    out = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--help"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--workload", "--probe", "--parity-seconds"):
        assert flag in out.stdout


def test_recording_words_are_rebuilt_from_the_pulled_pairs():
    """Host side of the recording pull: the (index, word) pairs the device listed, in any order, give back
    each population's array of bit words; the word index of a population starts at its base."""
    import types
    from genn_b200.runtime import Runtime
    rng = np.random.default_rng(5)
    shapes = {"a": (7, 1, 3), "b": (7, 2, 5)}
    arrays, layout, pairs, base = {}, {}, [], 0
    for name, shape in shapes.items():
        words = np.where(rng.random(shape) < 0.2, rng.integers(1, 2 ** 32, size=shape, dtype=np.uint64), 0).astype(np.uint32)
        arrays[name], layout[name] = words, (base, shape)
        idx = np.flatnonzero(words.reshape(-1))
        pairs += [(base + i, words.reshape(-1)[i]) for i in idx]
        base += words.size
    pairs = np.array(pairs, dtype=np.uint32)[rng.permutation(len(pairs))]
    fake = types.SimpleNamespace(_rec_pairs=pairs, _rec_layout=layout, _rec_host={})
    for name in shapes:
        assert np.array_equal(Runtime._recording_words(fake, name), arrays[name])
    # a recording that was copied whole is returned as it came
    fake = types.SimpleNamespace(_rec_pairs=None, _rec_layout={}, _rec_host=arrays)
    assert Runtime._recording_words(fake, "b") is arrays["b"]


def test_reference_arm_prints_the_contract_line_on_cpu():
    """`bench.py --impl reference` runs the reference's CPU backend (no GPU involved): one JSON line with the
    arm's keys, here on a hundredth of the network so that it ends in seconds."""
    res = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--ref-scale", "0.01",
                          "--steps", "1", "--warmup", "3", "--block", "100"],
                         capture_output=True, text=True, timeout=600, cwd=REPO)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["higher_is_better"] is True
    assert line["metric"].startswith("synaptic events/s") and line["unit"] == "synaptic events/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] == 1
    assert line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "0.01 s biological" in line["config"]["workload"]


def test_reference_arm_runs_on_rank_zero_only():
    """Launched one process per GPU, the arm is rank 0's work: every other rank leaves at once, silently."""
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    res = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                         capture_output=True, text=True, timeout=300, cwd=REPO, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""
