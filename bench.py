"""Benchmark: synaptic events per second and real-time factor of the
Potjans-Diesmann microcircuit architecture on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python bench.py --workload c2|c4|c5 [...]                  # the other configurations: E/I network, PROCEDURAL
                                                               # stress test, batched STDP with batch-reduce + all-reduce
    python bench.py --probe presyn|phases|e2e|dense [...]      # bounded single-kernel workloads (ncu, comparisons)

A bench STEP is a block of ``--block`` (default 1000) simulation time steps of
dt = 0.1 ms, i.e. 0.1 s of biological time, run by ONE launch of the persistent
time-step kernel.  At N GPUs the network has N times the neurons with the
published in-degrees (weak scaling) and each rank owns a contiguous slice of
every population's postsynaptic neurons together with their incoming synapses.

One JSON line is printed by rank 0.  ``value`` is whole-job synaptic events per
second with all state resident in HBM; ``e2e`` is the same metric through the
public ``GeNNModel`` API with the spike recording copied to page-locked host
memory every step; ``roofline`` is the persistent kernel of the timed region
(algorithmic bytes of the launch over its CUDA-event time) and
``roofline_saturated`` the SPARSE delivery kernel driven with a quarter of all
neurons spiking in one step (inputs far larger than L2); ``parity`` runs the x1
network the reference's CPU backend was run on (same arrays, drawn on the host),
split over the N GPUs, for 10 s and compares population firing rates and CV-ISI
with the reference's (tolerance 2 %); ``cpu_baseline`` times the
reference's own single-threaded CPU backend (or, where its build is absent and
labelled as such, the C port of its algorithm) on this box's host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

DT_MS = 0.1
ALGO_BYTES_PER_SPIKE = 8           # spike id + row length


def kernel_sources_digest() -> str:
    """SHA-256 over the kernel sources and the ABI headers: identifies the build a profiler
    figure was taken on."""
    import hashlib
    h = hashlib.sha256()
    for d in (os.path.join(REPO, "genn_b200", "csrc"), os.path.join(REPO, "include")):
        for name in sorted(os.listdir(d)):
            if name.endswith((".cu", ".cuh", ".h")):
                h.update(name.encode())
                h.update(open(os.path.join(d, name), "rb").read())
    return h.hexdigest()


def captured_traffic(kernel: str):
    """DRAM bytes per time step of `kernel` from the tracked record of an ncu capture
    (dram__bytes_read.sum + dram__bytes_write.sum of one short launch), or (None, why) when the
    record was taken on other kernel sources than the ones in the tree."""
    path = os.path.join(REPO, "profiles", "dram_traffic.txt")
    if not os.path.exists(path):
        return None, "no ncu capture recorded"
    digest = kernel_sources_digest()
    for line in open(path):
        f = line.split()
        if len(f) >= 5 and not line.startswith("#") and f[0] == kernel:
            if f[1] != digest:
                return None, "the recorded ncu capture was taken on other kernel sources"
            return (float(f[2]) + float(f[3])) / float(f[4]), f"ncu capture of a {f[4]}-step launch, scaled by the number of time steps"
    return None, "no ncu capture recorded for this kernel"


def measured_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled in a thread while the bench runs.

    NVML is read in-process every 5 ms (a bench step of this workload lasts a few milliseconds and
    nvidia-smi needs longer than the whole timed region to start); nvidia-smi is the fallback.
    Reading only: nothing is set."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []          # (time, sm MHz, max MHz, [reason names])
        self.proc = None
        self.thread = None
        self.running = False
        self.t_mark = 0.0
        self.source = None

    def _nvml_loop(self, handle, nvml):
        max_mhz = float(nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM))
        while self.running:
            try:
                mhz = float(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM))
                get = getattr(nvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or nvml.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = int(get(handle))
                self.rows.append((time.perf_counter(), mhz, max_mhz, [n for b, n in self.REASONS.items() if mask & b]))
            except Exception:
                pass
            time.sleep(0.005)

    def _smi_loop(self):
        for line in self.proc.stdout:
            r = [x.strip() for x in line.split(",")]
            if len(r) < 9:
                continue
            try:
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                self.rows.append((time.perf_counter(), float(r[1]), float(r[2]),
                                  [n for n, v in zip(names, r[5:9]) if v.lower().startswith("active")]))
            except ValueError:
                continue

    def start(self):
        self.running = True
        try:
            import pynvml as nvml
            nvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.gpu]) if visible and visible.split(",")[self.gpu].isdigit() else self.gpu
            handle = nvml.nvmlDeviceGetHandleByIndex(index)
            self.thread = threading.Thread(target=self._nvml_loop, args=(handle, nvml), daemon=True)
            self.thread.start()
            self.source = "nvml"
            return
        except Exception:
            pass
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._smi_loop, daemon=True)
            self.thread.start()
            self.source = "nvidia-smi"
        except Exception:
            self.proc = None

    def mark(self):
        """The timed region starts here; samples taken before it (the warm-up steps: the same kernel
        under the same load) are only used if the region is too short to catch one."""
        self.t_mark = time.perf_counter()

    def stop(self):
        t_end = time.perf_counter()
        self.running = False
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        if self.source is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source (NVML and nvidia-smi unavailable)"]}
        inside = [r for r in self.rows if self.t_mark <= r[0] <= t_end + (0.2 if self.proc is not None else 0.0)]
        window = "timed region"
        if not inside:
            inside, window = list(self.rows), "warm-up and timed region (the timed region was shorter than a sample)"
        reasons = sorted({n for r in inside for n in r[3]})
        return {"sm_mhz": float(np.median([r[1] for r in inside])) if inside else None,
                "sm_max_mhz": max(r[2] for r in inside) if inside else None,
                "reasons": reasons, "samples": len(inside), "window": window, "source": self.source}


def bytes_per_event(net) -> float:
    """Algorithmic HBM bytes per synaptic event, weighted by group size:
    index + weight (+ delay byte)."""
    tot, w = 0.0, 0.0
    for s in net.syns:
        n = float(net.pop(s.src).n) * s.row_stride
        b = np.dtype(s.ind_dtype).itemsize + (0 if s.wum == "CONST" else 4) + (1 if s.max_den_delay else 0)
        tot += n * b
        w += n
    return tot / w if w else 0.0


def run_reference_sample(scale: float, block: int, steps: int, warmup: int, seed: int = 1234):
    """Time the reference's own single_threaded_cpu backend (oracle/_ref, built
    from the unmodified reference sources) on a Potjans network with
    ``scale`` x the neurons and the published in-degrees.  Falls back to the C
    port of the same algorithm when the reference build is absent."""
    from genn_b200 import workloads
    from genn_b200.resolve import resolve, write_netspec
    model = workloads.potjans(neuron_scale=scale, seed=seed, host_connectivity=True, background="poisson", record=True)
    net = resolve(model)
    total_steps = (warmup + steps) * block
    driver = os.path.join(REPO, "oracle", "_ref", "ref_driver")
    out_deg = {p.name: np.zeros(p.n, dtype=np.int64) for p in net.pops}
    for s in net.syns:
        out_deg[s.src] += s.row_length
    if os.path.exists(driver):
        work = tempfile.mkdtemp(prefix="refarm_")
        try:
            spec = write_netspec(net, os.path.join(work, "spec"), total_steps, 0)
            os.makedirs(os.path.join(work, "out"))
            subprocess.check_call([driver, spec, os.path.join(work, "work"), os.path.join(work, "out")])
            timing = dict(l.split() for l in open(os.path.join(work, "out", "timing.txt")))
            seconds = float(timing["loop_seconds"])
            events = 0
            spikes = 0
            for p in net.pops:
                sp = np.fromfile(os.path.join(work, "out", f"spikes_{p.name}.bin"), dtype=np.uint32).reshape(-1, 2)
                events += int(out_deg[p.name][sp[:, 1]].sum())
                spikes += len(sp)
            kind = "reference"
        finally:
            shutil.rmtree(work, ignore_errors=True)
    else:
        from oracle.oracle import OracleRunner
        runner = OracleRunner(net, None)
        t0 = time.perf_counter()
        runner.step(total_steps)
        seconds = time.perf_counter() - t0
        events = runner.synaptic_events
        spikes = 0
        kind = "port"
        runner.close()
    sim_seconds = total_steps * DT_MS * 1e-3
    return {"kind": kind, "events": events, "spikes": spikes, "seconds": seconds,
            "events_per_s": events / seconds, "rtf": sim_seconds / seconds,
            "neurons": sum(p.n for p in net.pops), "synapses": int(sum(int(s.row_length.sum()) for s in net.syns)),
            "total_steps": total_steps}


def parity_leg(rank, world, device, block, seconds, all_reduce):
    """Statistics parity at the workload's size, at this N: the EXACT x1 network the reference's CPU
    backend was run on for tests/golden/stats_potjans_x1.json (same seed, connectivity, weights and
    delays drawn on the host by workloads.potjans), split over the `world` GPUs by target neuron,
    simulated for `seconds` with spike recording.  Per-population firing rate and CV-ISI are compared
    with the reference's.  (The timed network is drawn on the device from another seed, and a
    different draw of the connectivity alone moves the population rates by up to 3 %: only the same
    network can be held to 2 %.)  Every rank decodes the slice of each population it updates; the
    partial sums are combined across ranks."""
    from genn_b200 import stats, workloads
    path = os.path.join(REPO, "tests", "golden", "stats_potjans_x1.json")
    if not os.path.exists(path):
        return {"ok": None, "note": "no reference statistics on disk"}
    golden = json.load(open(path))
    want = golden["populations"]
    t0 = time.perf_counter()
    shard = (rank, world) if world > 1 else None
    model = workloads.potjans(neuron_scale=1.0, seed=int(golden.get("seed", 2024)), host_connectivity=True,
                              background="poisson", record=True, shard=shard)
    model.build()
    model.load(num_recording_timesteps=block, device=device, shard=shard)
    rt = model._runtime
    net = rt.net
    build_s = time.perf_counter() - t0
    blocks = max(1, int(round(seconds / (block * DT_MS * 1e-3))))
    spikes = {p.name: ([], []) for p in net.pops}
    t0 = time.perf_counter()
    for _ in range(blocks):
        model.step_time(block)
        model.pull_recording_buffers_from_device()
        for p in net.pops:
            times, ids = rt.recorded_spikes(p.name)[0]
            spikes[p.name][0].append(np.rint(times / net.dt).astype(np.int64))
            spikes[p.name][1].append(ids)
    run_s = time.perf_counter() - t0
    names = [p.name for p in net.pops]
    sums = np.zeros((len(names), 4))
    for j, p in enumerate(net.pops):
        lo, hi = (p.shard_bounds[rank], p.shard_bounds[rank + 1]) if shard else (0, p.n)
        sums[j] = stats.partial(np.concatenate(spikes[p.name][0]), np.concatenate(spikes[p.name][1]), hi - lo, first_id=lo)
    schedule = rt.schedule
    model.unload()
    if all_reduce is not None:
        import torch
        t = torch.tensor(sums, dtype=torch.float64, device="cuda")
        all_reduce(t)
        sums = t.cpu().numpy()
    duration = blocks * block * DT_MS * 1e-3
    got = {n: stats.merge([sums[j]], duration) for j, n in enumerate(names)}
    rate_err, cv_err = stats.compare(got, want)
    return {"rates_max_rel_err": rate_err, "cv_isi_max_rel_err": cv_err, "tolerance": 0.02,
            "ok": bool(rate_err <= 0.02 and cv_err <= 0.02), "simulated_seconds": duration,
            "network": f"Potjans x1, seed {int(golden.get('seed', 2024))}, host-drawn connectivity: the reference's own network, "
                       f"sharded over {world} GPU(s)",
            "schedule": int(schedule), "build_seconds": round(build_s, 1), "run_seconds": round(run_s, 1),
            "rates_hz": {n: round(got[n]["rate_hz"], 4) for n in names},
            "reference_rates_hz": {n: round(want[n]["rate_hz"], 4) for n in names},
            "cv_isi": {n: round(got[n]["cv_isi"], 4) for n in names},
            "reference_cv_isi": {n: round(want[n]["cv_isi"], 4) for n in names},
            "note": "reference: GeNN single_threaded_cpu backend on the identical network, 10 s simulated "
                    "(chaotic network: statistics, not spike trains, are comparable)"}


def reference_arm(args):
    """--impl reference: the reference's CPU implementation of the path on this
    box's host cores (single-threaded by construction)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = run_reference_sample(args.ref_scale, args.block, args.steps, args.warmup)
    steps_total = args.warmup + args.steps
    ms_per_step = r["seconds"] / steps_total * 1e3
    line = {
        "impl": "reference", "metric": "synaptic events/s (Potjans microcircuit architecture)",
        "value": r["events_per_s"], "unit": "synaptic events/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "realtime_factor": r["rtf"],
        "config": {"workload": f"Potjans-Diesmann microcircuit architecture x{args.ref_scale:g}: {r['neurons']} LIF neurons, "
                               f"published in-degrees ({r['synapses']} synapses, drawn on the host), SPARSE with dendritic "
                               f"delays, PoissonExp background, dt=0.1 ms; one bench step = {args.block} time steps "
                               f"({args.block * 1e-4:g} s biological)",
                   "parallelism": "the reference's CPU backend is single-threaded; at N > 1 it runs the x1 network "
                                  "(a bounded sample of the xN workload: same in-degrees, same per-neuron work)",
                   "timing": "wall clock around the reference's stepTime loop (all warm-up and timed steps)"},
        "cpu_baseline": {"value": r["events_per_s"], "unit": "synaptic events/s", "cores": 1, "kind": r["kind"],
                         "sample": f"neuron_scale={args.ref_scale}, {r['total_steps']} time steps"},
        "e2e": {"value": r["events_per_s"], "unit": "synaptic events/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_c2(args):
    """Recurrent conductance-based E/I network (80 000 + 20 000 LIF, fixed in-degree 1 000: 100 M synapses with constant
    weights, 4 B per event; ExpCond, 1 ms axonal delay, dt = 0.1 ms), single GPU.  One bench step = --block time steps."""
    import torch
    from genn_b200 import workloads
    torch.cuda.set_device(0)
    block = args.block
    model = workloads.cond_ei(neuron_scale=1.0, record=True)
    model.build()
    model.load(num_recording_timesteps=block, device=0)
    rt = model._runtime
    rt.set_option("count_events", 1)
    for item in args.option:
        opt_name, opt_value = item.split("=")
        rt.set_option(opt_name, float(opt_value))
    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(args.warmup):
        rt.step_time(block)
    rt.synchronize()
    ev0, sp0, l0 = rt.counter("synaptic_events"), rt.counter("spikes"), rt.kernel_launches
    sampler.mark()
    ms = rt.step_time_timed(args.steps * block)
    clocks = sampler.stop()
    ev1, sp1, l1 = rt.counter("synaptic_events"), rt.counter("spikes"), rt.kernel_launches
    seconds, sim_seconds = ms * 1e-3, args.steps * block * DT_MS * 1e-3
    model.step_time(block)
    model.pull_recording_buffers_from_device()
    e0, moved0 = rt.counter("synaptic_events"), rt.factory.d2h_bytes
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.step_time(block)
        model.pull_recording_buffers_from_device()
    e2e_s = time.perf_counter() - t0
    d2h = (rt.factory.d2h_bytes - moved0) / max(1, args.steps)      # what the pulls moved (non-zero recording words as pairs)
    e2e_ev = rt.counter("synaptic_events") - e0
    n = sum(p.n for p in rt.net.pops)
    bytes_algo = (ev1 - ev0) * bytes_per_event(rt.net) + (sp1 - sp0) * ALGO_BYTES_PER_SPIKE
    hbm_peak, peak_kind = measured_peaks()
    line = {"metric": "synaptic events/s (recurrent conductance-based E/I network)", "value": (ev1 - ev0) / seconds,
            "unit": "synaptic events/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "realtime_factor": sim_seconds / seconds, "us_per_timestep": ms * 1e3 / (args.steps * block),
            "config": {"workload": f"{n} LIF neurons (80 % excitatory), fixed in-degree 1000 drawn on the host, constant weights "
                                   f"0.6 / 6.7 nS, ExpCond, 1 ms axonal delay, constant drive 0.35 nA, dt = 0.1 ms; one bench step = "
                                   f"{block} time steps",
                       "schedule": int(rt.schedule), "step_path": rt.step_path()[0],
                       "mean_rate_hz": (sp1 - sp0) / n / sim_seconds, "bytes_per_event": bytes_per_event(rt.net),
                       "l2": "400 MB of synapse indices, larger than L2"},
            "clocks": clocks,
            "e2e": {"value": e2e_ev / e2e_s, "unit": "synaptic events/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(l1 - l0),
            "roofline": {"kernel": "persistent step kernel" if rt.step_path()[0] else "per-kernel path", "bound": "hbm",
                         "achieved": bytes_algo / seconds / 1e9, "peak": hbm_peak, "unit": "GB/s",
                         "frac": bytes_algo / seconds / 1e9 / hbm_peak, "traffic": None, "peak_source": peak_kind,
                         "algorithmic_bytes_per_launch": bytes_algo,
                         "note": "natural firing rates (3 Hz): a step is latency, not bandwidth"}}
    print(json.dumps(line), flush=True)
    model.unload()


def run_c4(args):
    """PROCEDURAL connectivity stress test (single GPU): nothing of the ~1e9-synapse matrix is stored,
    every spike regenerates its row and weights.  One bench step = --block time steps of 1 ms (default
    100).  Every synapse is one floating-point reduction into L2 and no HBM traffic: the figures of
    merit are synaptic events/s and L2 reductions/s (the same number)."""
    import torch
    from genn_b200 import workloads
    torch.cuda.set_device(0)
    block = args.block if args.block != 1000 else 100
    model = workloads.procedural_stress(num_neurons=args.c4_neurons, threads_per_spike=args.c4_threads, record=True)
    model.build()
    model.load(num_recording_timesteps=block, device=0)
    rt = model._runtime
    rt.set_option("count_events", 1)
    for item in args.option:
        opt_name, opt_value = item.split("=")
        rt.set_option(opt_name, float(opt_value))
    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(args.warmup):
        rt.step_time(block)
    rt.synchronize()
    ev0, sp0, l0 = rt.counter("synaptic_events"), rt.counter("spikes"), rt.kernel_launches
    sampler.mark()
    ms = rt.step_time_timed(args.steps * block)
    clocks = sampler.stop()
    ev1, sp1, l1 = rt.counter("synaptic_events"), rt.counter("spikes"), rt.kernel_launches
    seconds = ms * 1e-3
    sim_seconds = args.steps * block * 1e-3
    # the presynaptic kernel alone, per launch (CUDA event pairs)
    rt.enable_timing(True)
    rt.reset_timers()
    tev0 = rt.counter("synaptic_events")
    rt.step_time(block)
    rt.synchronize()
    tev = rt.counter("synaptic_events") - tev0
    pre_s, neu_s = rt.timer("presynaptic_update"), rt.timer("neuron_update")
    rt.enable_timing(False)
    # end to end: steps plus the spike recording pulled into page-locked memory
    model.step_time(block)
    model.pull_recording_buffers_from_device()
    e0, moved0 = rt.counter("synaptic_events"), rt.factory.d2h_bytes
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.step_time(block)
        model.pull_recording_buffers_from_device()
    e2e_s = time.perf_counter() - t0
    d2h = (rt.factory.d2h_bytes - moved0) / max(1, args.steps)      # what the pulls moved (non-zero recording words as pairs)
    e2e_ev = rt.counter("synaptic_events") - e0
    n = sum(p.n for p in rt.net.pops)
    line = {"metric": "synaptic events/s (PROCEDURAL connectivity stress test)", "value": (ev1 - ev0) / seconds,
            "unit": "synaptic events/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "realtime_factor": sim_seconds / seconds,
            "config": {"workload": f"{n} LIF neurons, recurrent PROCEDURAL FixedProbability p=0.001, weights Normal(0.1, 0.01) nA "
                                   f"regenerated per spike, Poisson drive 5 Hz onto 10 % of the neurons, dt = 1 ms; one bench "
                                   f"step = {block} time steps",
                       "threads_per_spike": args.c4_threads,
                       "mean_rate_hz": (sp1 - sp0) / n / sim_seconds,
                       "l2": "no synapse data exists; the reductions' targets (4 MB per postsynaptic buffer) live in L2"},
            "clocks": clocks,
            "e2e": {"value": e2e_ev / e2e_s, "unit": "synaptic events/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(l1 - l0),
            "l2_reductions_per_s": (ev1 - ev0) / seconds,
            "roofline": {"kernel": "presynapticProceduralKernel", "bound": "hbm", "achieved": 0.0, "peak": measured_peaks()[0],
                         "unit": "GB/s", "frac": 0.0, "traffic": None,
                         "launches": block, "avg_launch_us": pre_s / block * 1e6, "neuron_kernel_avg_launch_us": neu_s / block * 1e6,
                         "events_per_s_in_kernel": tev / pre_s if pre_s > 0 else None,
                         "note": "0 algorithmic HBM bytes per event: the kernel is bound by Philox + log arithmetic and by "
                                 "L2 reductions (events_per_s_in_kernel = reductions/s inside the presynaptic kernel)"}}
    print(json.dumps(line), flush=True)
    model.unload()


def run_c5(args):
    """Batched plasticity, data-parallel over the GPUs: every rank holds --c5-batch copies of the dynamic
    state (own Poisson draws, own weights), connectivity replicated.  One bench step = 100 time steps of
    1 ms followed by the custom update group "gradient": sum of the weights over the batch (batchReduceKernel),
    ONE NCCL all-reduce of the packed sums over the ranks, mean written back into every copy.  `value` =
    synaptic events/s of the whole job (pre-side and post-side STDP events); `roofline` = the batch-reduce
    kernels (4 B x batch read + 4 B target + 4 B x batch written back per synapse slot)."""
    import torch
    import torch.distributed as dist
    from genn_b200 import workloads
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    block = 100
    model, sg = workloads.batched_stdp(num_pre=args.c5_neurons, num_post=args.c5_neurons, batch=args.c5_batch,
                                       seed=55 + rank, world=world)
    model.seed = 55                      # the same connectivity on every rank; the state differs through the batch streams
    model.build()
    model.load(device=local_rank)
    rt = model._runtime
    rt.set_option("count_events", 1)
    if world > 1:
        rt.init_data_parallel(rank, world)
    hbm_peak, peak_kind = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def allreduce(value, op):
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=op)
        return float(t.item())

    def bench_step():
        rt.step_time(block)
        rt.custom_update("gradient")

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        bench_step()
    rt.synchronize()
    ev0, l0 = rt.counter("synaptic_events"), rt.kernel_launches
    barrier()
    sampler.mark()
    rt.timed_begin()
    for _ in range(args.steps):
        bench_step()
    ms = rt.timed_end()
    barrier()
    clocks = sampler.stop()
    ev1, l1 = rt.counter("synaptic_events"), rt.kernel_launches
    ms = allreduce(ms, dist.ReduceOp.MAX if world > 1 else None)
    events = allreduce(float(ev1 - ev0), dist.ReduceOp.SUM if world > 1 else None)
    # the custom update alone (CUDA event pair around reduce + all-reduce + write-back)
    rt.enable_timing(True)
    rt.reset_timers()
    reps = 5
    for _ in range(reps):
        barrier()
        rt.custom_update("gradient")
    rt.synchronize()
    cu_s = allreduce(rt.timer("custom_update_gradient") / reps, dist.ReduceOp.MAX if world > 1 else None)
    # ... and the kernels of a time step (a CUDA event pair around every launch)
    rt.reset_timers()
    sp0, pe0 = rt.counter("spikes"), rt.counter("synaptic_events")
    rt.step_time(block)
    rt.synchronize()
    kernel_us = {n: rt.timer(n) / block * 1e6 for n in ("neuron_update", "presynaptic_update", "postsynaptic_update")}
    spikes_per_step = (rt.counter("spikes") - sp0) / block
    pre_events_per_step = (rt.counter("synaptic_events") - pe0) / block
    rt.enable_timing(False)
    slots = int(np.prod(rt.plan.arrays["syn.g"].shape[1:], dtype=np.int64))
    # read the batch, write the target, write the batch back (+ the packed buffer written and read when ranks combine)
    cu_bytes = slots * (4.0 * args.c5_batch + 4.0 + 4.0 * args.c5_batch + (8.0 if world > 1 else 0.0))
    # end to end: the same steps plus the reduced weights pulled to the host after every update
    red = model.custom_updates["mean_g"].vars["reduction"]
    bench_step()
    red.pull_from_device()
    barrier()
    t0 = time.perf_counter()
    e0 = rt.counter("synaptic_events")
    for _ in range(args.steps):
        bench_step()
        red.pull_from_device()
    barrier()
    e2e_s = allreduce(time.perf_counter() - t0, dist.ReduceOp.MAX if world > 1 else None)
    e2e_ev = allreduce(float(rt.counter("synaptic_events") - e0), dist.ReduceOp.SUM if world > 1 else None)
    if rank == 0:
        seconds = ms * 1e-3
        line = {"metric": "synaptic events/s (batched STDP, data-parallel)", "value": events / seconds, "unit": "synaptic events/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "realtime_factor": args.steps * block * 1e-3 / seconds,
                "config": {"workload": f"{args.c5_neurons} Poisson inputs (25 Hz) -> {args.c5_neurons} LIF, SPARSE p=0.1 ({slots} synapse "
                                       f"slots), additive STDP, {args.c5_batch} batch entries per GPU x {world} GPU(s); one bench step = "
                                       f"{block} time steps of 1 ms + batch-reduce custom update with one packed NCCL all-reduce",
                           "parallelism": f"data-parallel over {world} GPU(s), connectivity replicated",
                           "kernel_us_per_time_step": kernel_us, "spikes_per_time_step": spikes_per_step,
                           "presynaptic_events_per_time_step": pre_events_per_step,
                           "l2": f"weights: {slots * 4 * args.c5_batch / 1e9:.2f} GB per GPU, larger than L2"},
                "clocks": clocks,
                "e2e": {"value": e2e_ev / e2e_s, "unit": "synaptic events/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": slots * 4},
                "gpu_launches": int(l1 - l0),
                "roofline": {"kernel": "batchReduceKernel (reduce, all-reduce, write back)", "bound": "hbm",
                             "achieved": cu_bytes / cu_s / 1e9, "peak": hbm_peak, "unit": "GB/s", "frac": cu_bytes / cu_s / 1e9 / hbm_peak,
                             "traffic": None, "peak_source": peak_kind, "launches": reps, "avg_launch_ms": cu_s * 1e3,
                             "algorithmic_bytes_per_launch": cu_bytes,
                             "all_reduce_bytes": slots * 4,
                             "note": "CUDA events around the whole custom update: two kernels and the all-reduce between them"}}
        print(json.dumps(line), flush=True)
    model.unload()
    if world > 1:
        dist.destroy_process_group()


def run_probe(args):
    """Bounded single-kernel workloads, sized for a profiler capture that ends by itself.

    presyn: Potjans architecture at --probe-scale (default 0.5) times the neurons (in-degrees and
            therefore row lengths unchanged), --probe-fraction of every population marked as having
            spiked, --probe-reps launches of the presynaptic update.  The device holds about
            2.6 GB x scale; one launch reads about scale x fraction x 2.1 GB (twice L2 at the defaults).
    phases: --probe-warm + --probe-steps time steps of the persistent kernel at natural rates with its
            clock64 phase counters on.
    e2e:    where one GeNNModel.step_time + recording pull spends its time.
    dense:  batched DENSE presynaptic update, this library's row gather beside the same update as a contraction
            through the vendor GEMM (8192 x 8192 weights, batch 1 / 32 / 256)."""
    from genn_b200 import workloads
    from genn_b200.runtime import Runtime
    if args.probe == "presyn":
        scale = args.probe_scale if args.probe_scale is not None else 0.5
        model = workloads.potjans(neuron_scale=scale, seed=1234)
        model.build()
        rt = Runtime(model, None)
        net = rt.net
        for item in args.option:
            k, v = item.split("=")
            rt.set_option(k, float(v))
        rng = np.random.default_rng(99)
        out_deg = {}
        for s in net.syns:
            out_deg[s.src] = out_deg.get(s.src, 0) + rt.array(f"{s.name}.row_length").astype(np.int64)
        events = spikes = 0
        for p in net.pops:
            ids = np.sort(rng.choice(p.n, size=max(1, int(p.n * args.probe_fraction)), replace=False)).astype(np.uint32)
            rt.set_spike_list(p.name, ids)
            events += int(out_deg[p.name][ids].sum()) if p.name in out_deg else 0
            spikes += len(ids)
        for _ in range(2):
            rt.update_synapses()
        rt.enable_timing(True)
        rt.reset_timers()
        for _ in range(args.probe_reps):
            rt.update_synapses()
        rt.synchronize()
        sec = rt.timer("presynaptic_update") / args.probe_reps
        bpe = bytes_per_event(net)
        out = {"probe": "presyn", "scale": scale, "fraction": args.probe_fraction,
               "events_per_launch": events, "spikes_per_launch": spikes, "launch_ms": sec * 1e3,
               "events_per_s": events / sec, "bytes_per_event": bpe,
               "GBps": (events * bpe + spikes * ALGO_BYTES_PER_SPIKE) / sec / 1e9}
        if any(item.startswith("fused_profile=") for item in args.option):
            # the tiled kernel's own clock64 record of its last launch, per CTA: [min, median, max]
            cyc = rt.cta_cycles()
            rows = np.stack([cyc[:, 0], cyc[:, 1], cyc[:, 2] >> np.uint64(32), cyc[:, 2] & np.uint64(0xFFFFFFFF), cyc[:, 3]], axis=1).astype(np.int64)
            out["tiled_cta_columns"] = ["cycles", "cycles_outside_ticket_loops", "segments", "tickets", "cycles_idle_at_loop_ends"]
            out["tiled_cta_rows_by_cycles"] = rows[np.argsort(rows[:, 0])].tolist()
        print(json.dumps(out))
        rt.close()
    elif args.probe == "dense":
        # Batched DENSE presynaptic update: this library's row gather (4 x numPost bytes per spike and batch
        # entry) beside the same update written as a contraction, spikes[B x numPre] (0/1) @ W[numPre x numPost],
        # on the tensor cores through the vendor GEMM (comparison only: it reads all of W whatever the activity)
        import torch
        from genn_b200 import GeNNModel, init_postsynaptic, init_var, init_weight_update
        n, rows = args.probe_dense_size, []
        for batch in (1, 32, 256):
            m = GeNNModel("float", "dense_probe")
            m.dt = 1.0
            m.batch_size = batch
            src = m.add_neuron_population("pre", n, "Poisson", {"rate": 25.0}, {"timeStepToSpike": 0.0})
            lif = {"C": 40.0, "TauM": 20.0, "Vrest": -65.0, "Vreset": -70.0, "Vthresh": -55.0, "Ioffset": 0.0, "TauRefrac": 2.0}
            trg = m.add_neuron_population("post", n, "LIF", lif, {"V": -65.0, "RefracTime": 0.0})
            m.add_synapse_population("syn", "DENSE", src, trg,
                                     init_weight_update("StaticPulse", {}, {"g": init_var("Uniform", {"min": 0.0, "max": 0.01})}),
                                     init_postsynaptic("ExpCurr", {"tau": 5.0}))
            m.build()
            rt = Runtime(m, None)
            rng = np.random.default_rng(5)
            active = max(1, int(n * args.probe_fraction))
            spikes = torch.zeros((batch, n), dtype=torch.bfloat16, device="cuda")
            for b in range(batch):
                ids = np.sort(rng.choice(n, size=active, replace=False)).astype(np.uint32)
                rt.set_spike_list("pre", ids, batch=b)
                spikes[b, torch.from_numpy(ids.astype(np.int64)).cuda()] = 1
            for _ in range(2):
                rt.update_synapses()
            rt.enable_timing(True)
            rt.reset_timers()
            for _ in range(args.probe_reps):
                rt.update_synapses()
            rt.synchronize()
            gather_s = rt.timer("presynaptic_update") / args.probe_reps
            rt.close()
            w16 = torch.rand((n, n), device="cuda").to(torch.bfloat16)
            w32 = torch.rand((n, n), device="cuda")
            s32 = spikes.float()
            out = {}
            for name, a, w in (("bf16", spikes, w16), ("tf32", s32, w32)):
                torch.backends.cuda.matmul.allow_tf32 = True
                for _ in range(3):
                    torch.matmul(a, w)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.probe_reps):
                    torch.matmul(a, w)
                e1.record()
                torch.cuda.synchronize()
                out[name] = e0.elapsed_time(e1) / args.probe_reps * 1e-3
            rows.append({"batch": batch, "active_rows_per_batch_entry": active,
                         "gather_us": gather_s * 1e6, "gather_GBps": batch * active * 4.0 * n / gather_s / 1e9,
                         "gemm_bf16_us": out["bf16"] * 1e6, "gemm_tf32_us": out["tf32"] * 1e6,
                         "gemm_bf16_TFLOPs": 2.0 * batch * n * n / out["bf16"] / 1e12})
            del w16, w32, spikes, s32
        print(json.dumps({"probe": "dense", "num_pre": n, "num_post": n, "fraction": args.probe_fraction, "rows": rows}))
    elif args.probe == "phases":
        scale = args.probe_scale if args.probe_scale is not None else 1.0
        model = workloads.potjans(neuron_scale=scale, seed=1234, min_delay=args.min_delay,
                                  extra_delay_slots=1 if args.min_delay > 0 else 0)
        model.build()
        rt = Runtime(model, None)
        for item in args.option:
            k, v = item.split("=")
            rt.set_option(k, float(v))
        rt.step_time(args.probe_warm)
        rt.synchronize()
        rt.set_option("fused_profile", 1)
        names = ["cycles_presynaptic", "cycles_barrier_a", "cycles_neuron", "cycles_barrier_b"]
        before = [rt.counter(n) for n in names]
        ms = rt.step_time_timed(args.probe_steps)
        after = [rt.counter(n) for n in names]
        out = {"probe": "phases", "scale": scale, "steps": args.probe_steps, "us_per_step": ms * 1e3 / args.probe_steps,
               "step_path": rt.step_path(), "schedule": rt.schedule, "stream_warps": rt.counter("stream_warps")}
        for n, a, b in zip(names, before, after):
            out[n + "_per_step"] = (b - a) / args.probe_steps
        print(json.dumps(out))
        rt.close()
    else:
        scale = args.probe_scale if args.probe_scale is not None else 1.0
        model = workloads.potjans(neuron_scale=scale, seed=1234, record=True)
        model.build()
        model.load(num_recording_timesteps=args.block)
        rt = model._runtime
        rt.step_time(3 * args.block)
        rt.synchronize()
        kernel_ms = [rt.step_time_timed(args.block) for _ in range(args.probe_reps)]
        launch_s, sync_s, pull_s = [], [], []
        for _ in range(args.probe_reps):
            t0 = time.perf_counter()
            model.step_time(args.block)
            t1 = time.perf_counter()
            rt.synchronize()
            t2 = time.perf_counter()
            model.pull_recording_buffers_from_device()
            t3 = time.perf_counter()
            launch_s.append(t1 - t0)
            sync_s.append(t2 - t1)
            pull_s.append(t3 - t2)
        print(json.dumps({"probe": "e2e", "block": args.block, "kernel_ms_per_block": kernel_ms,
                          "launch_call_ms": [x * 1e3 for x in launch_s], "wait_ms": [x * 1e3 for x in sync_s],
                          "pull_ms": [x * 1e3 for x in pull_s]}))
        model.unload()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--block", type=int, default=1000, help="simulation time steps per bench step")
    ap.add_argument("--ref-scale", type=float, default=1.0,
                    help="--impl reference: neuron scale of the network the reference runs (1 = the bench's own x1 workload; "
                         "smaller values for quick runs)")
    ap.add_argument("--cpu-sample-scale", type=float, default=0.05,
                    help="neuron scale of the bounded cpu_baseline sample inside the GPU arm's run")
    ap.add_argument("--parity-seconds", type=float, default=10.0,
                    help="simulated seconds of the rate / CV-ISI comparison with the reference's statistics (0: skip)")
    ap.add_argument("--probe-dense-size", type=int, default=8192)
    ap.add_argument("--probe", choices=["presyn", "phases", "e2e", "dense"], default=None,
                    help="run a bounded single-kernel workload (for profiling) instead of the benchmark")
    ap.add_argument("--workload", choices=["potjans", "c2", "c4", "c5"], default="potjans",
                    help="potjans: the headline workload; c2: recurrent conductance-based E/I network (80 k + 20 k LIF, "
                         "in-degree 1000, 1 ms axonal delay; single GPU); c4: the PROCEDURAL connectivity stress test (1 M LIF neurons, "
                         "p = 0.001, dt = 1 ms; single GPU); c5: batched plasticity (10 k Poisson -> 10 k LIF, STDP, 32 batch "
                         "entries per GPU, batch-reduce + all-reduce every 100 steps)")
    ap.add_argument("--c5-batch", type=int, default=32, help="batch entries per GPU")
    ap.add_argument("--c5-neurons", type=int, default=10000)
    ap.add_argument("--c4-neurons", type=int, default=1_000_000)
    ap.add_argument("--c4-threads", type=int, default=32, help="threads that share one regenerated row")
    ap.add_argument("--probe-scale", type=float, default=None)
    ap.add_argument("--probe-fraction", type=float, default=0.25)
    ap.add_argument("--probe-steps", type=int, default=2000)
    ap.add_argument("--probe-warm", type=int, default=2000)
    ap.add_argument("--probe-reps", type=int, default=3)
    ap.add_argument("--neuron-scale", type=float, default=None, help="override the workload size (debugging)")
    ap.add_argument("--min-delay", type=float, default=0.0,
                    help="lower clip of the delay distribution in ms (0: the reference script's; not the headline if changed)")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="runner option to set before timing (experiments; see b200_set_option)")
    ap.add_argument("--sharded-emit", action="store_true",
                    help="N > 1: spiking threads push their nearest synapses into the other GPUs' rings (experiment)")
    ap.add_argument("--cpu-sample-blocks", type=int, default=100,
                    help="length of the CPU baseline sample in bench steps (1000 time steps each) at --ref-scale")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-saturated", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.probe:
        run_probe(args)
        return
    if args.workload == "c2":
        run_c2(args)
        return
    if args.workload == "c4":
        run_c4(args)
        return
    if args.workload == "c5":
        run_c5(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run, one rank per GPU")
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from genn_b200 import workloads
    from genn_b200.resolve import resolve
    from genn_b200.runtime import Runtime

    scale = args.neuron_scale if args.neuron_scale is not None else float(world)
    block = args.block
    hbm_peak, peak_kind = measured_peaks()

    # ---- build through the public API ---------------------------------------------
    model = workloads.potjans(neuron_scale=scale, seed=1234, record=True,
                              shard=(rank, world) if world > 1 else None,
                              min_delay=args.min_delay, extra_delay_slots=1 if args.min_delay > 0 else 0)
    model.build()
    model.load(num_recording_timesteps=block, device=local_rank, shard=(rank, world) if world > 1 else None,
               sharded_emit=(True if args.sharded_emit else None))
    rt = model._runtime
    net = rt.net
    rt.set_option("count_events", 1)
    rt.set_option("graph_steps", min(block, 100))
    for item in args.option:
        opt_name, opt_value = item.split("=")
        rt.set_option(opt_name, float(opt_value))
    bpe = bytes_per_event(net)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def allreduce(value, op):
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=op)
        return float(t.item())

    # ---- device-resident throughput: W warm-up, K timed steps -------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        rt.step_time(block)
    rt.synchronize()
    ev0, sp0, l0 = rt.counter("synaptic_events"), rt.counter("spikes"), rt.kernel_launches
    barrier()
    sampler.mark()
    ms = rt.step_time_timed(args.steps * block)        # CUDA events on the runner's own stream
    barrier()
    clocks = sampler.stop()
    ev1, sp1, l1 = rt.counter("synaptic_events"), rt.counter("spikes"), rt.kernel_launches
    ms = allreduce(ms, dist.ReduceOp.MAX if world > 1 else None)
    events = allreduce(float(ev1 - ev0), dist.ReduceOp.SUM if world > 1 else None)
    spikes = allreduce(float(sp1 - sp0), dist.ReduceOp.SUM if world > 1 else None)
    seconds = ms * 1e-3
    sim_seconds = args.steps * block * DT_MS * 1e-3
    value = events / seconds

    # ---- end to end through the public API: step + recording to pinned host memory ---
    d2h = sum(a.nbytes for n, a in rt.plan.arrays.items() if n.endswith(".record"))
    # (one untimed round first: the first pull allocates the page-locked host buffers)
    model.step_time(block)
    model.pull_recording_buffers_from_device()
    e2e_ev0 = rt.counter("synaptic_events")
    d2h0 = rt.factory.d2h_bytes
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.step_time(block)
        model.pull_recording_buffers_from_device()
    barrier()
    # what the pulls really moved: the recording's non-zero words as (index, word) pairs
    d2h_moved = allreduce(float(rt.factory.d2h_bytes - d2h0) / max(1, args.steps), dist.ReduceOp.SUM if world > 1 else None)
    d2h = allreduce(float(d2h), dist.ReduceOp.SUM if world > 1 else None)      # (whole job: every process pulls its slice)
    e2e_seconds = allreduce(time.perf_counter() - t0, dist.ReduceOp.MAX if world > 1 else None)
    e2e_events = allreduce(float(rt.counter("synaptic_events") - e2e_ev0), dist.ReduceOp.SUM if world > 1 else None)
    # firing rates from the last pulled recording (sanity: the network is in its asynchronous state)
    rates = {}
    for p in net.pops:
        t_, ids = rt.recorded_spikes(p.name)[0]
        n_local = rt.plan.neuron_descs[[q.name for q in net.pops].index(p.name)].num_update
        rates[p.name] = round(len(ids) / max(1, n_local) / (block * DT_MS * 1e-3), 3)

    # ---- where a step's time goes inside the persistent kernel (clock64 per phase, CTA 0) ---
    probe_steps = min(args.steps * block, 2000)
    rt.set_option("fused_profile", 1)
    names = ["cycles_presynaptic", "cycles_barrier_a", "cycles_neuron", "cycles_barrier_b"] + [f"probe{i}" for i in range(12)]
    before = [rt.counter(n) for n in names]
    pev0, psp0 = rt.counter("synaptic_events"), rt.counter("spikes")
    barrier()
    rt.step_time(probe_steps)
    rt.synchronize()
    barrier()
    pev, psp = rt.counter("synaptic_events") - pev0, rt.counter("spikes") - psp0
    phase_cycles = {n: (rt.counter(n) - b) / probe_steps for n, b in zip(names, before)}
    cta = rt.cta_cycles().astype(np.float64) / probe_steps
    if len(cta):
        # spike-header wait (counts and first ids of every source) inside the presynaptic phase, per CTA
        head = np.asarray(rt.header_cycles, dtype=np.float64) / probe_steps
        phase_cycles["header_median"] = float(np.median(head))
        phase_cycles["header_max"] = float(head.max())
        phase_cycles["cta_presynaptic_min_median_max"] = [float(cta[:, 0].min()), float(np.median(cta[:, 0])),
                                                          float(cta[:, 0].max())]
        phase_cycles["cta_neuron_min_median_max"] = [float(cta[:, 2].min()), float(np.median(cta[:, 2])), float(cta[:, 2].max())]
        phase_cycles["cta_header_or_arrival_min_median_max"] = [float(head.min()), float(np.median(head)), float(head.max())]
        phase_cycles["cta_latest"] = int(np.argmax(head))
    rt.set_option("fused_profile", 0)
    sm_hz = (clocks.get("sm_mhz") or 1965.0) * 1e6

    # ---- roofline of the presynaptic kernel, live, per-kernel CUDA events ---------------
    if world == 1:
        rt.enable_timing(True)
        rt.reset_timers()
        tev0, tsp0 = rt.counter("synaptic_events"), rt.counter("spikes")
        rt.step_time(probe_steps)
        rt.synchronize()
        tev, tsp = rt.counter("synaptic_events") - tev0, rt.counter("spikes") - tsp0
        pre_s, neu_s = rt.timer("presynaptic_update"), rt.timer("neuron_update")
        rt.enable_timing(False)
        nat_bytes = tev * bpe + tsp * ALGO_BYTES_PER_SPIKE
        nat_gbs = nat_bytes / pre_s / 1e9 if pre_s > 0 else 0.0
        per_kernel = {"kernel": "presynapticSparseKernel", "achieved": nat_gbs, "unit": "GB/s", "frac": nat_gbs / hbm_peak,
                      "launches": probe_steps, "avg_launch_us": pre_s / probe_steps * 1e6,
                      "neuron_kernel_avg_launch_us": neu_s / probe_steps * 1e6,
                      "algorithmic_bytes_per_launch": nat_bytes / probe_steps,
                      "note": "the one-launch-per-kernel path at the same firing rates (CUDA event pair around every launch)"}
        # the kernel of the timed region: ONE persistent launch runs all its time steps
        launch_bytes = float(ev1 - ev0) * bpe + float(sp1 - sp0) * ALGO_BYTES_PER_SPIKE
        launch_gbs = launch_bytes / seconds / 1e9
        timed_steps = args.steps * block
        per_step, traffic_note = (captured_traffic("streamStepKernel")
                                  if (scale == 1.0 and args.min_delay == 0.0 and rt.schedule == 3)
                                  else (None, "no capture for this configuration"))
        traffic = per_step * timed_steps if per_step is not None else None
        roofline = {"kernel": ["fusedStepKernel", "fusedStepKernel", "fusedStepKernel", "streamStepKernel"][rt.schedule]
                              + f" (persistent: {timed_steps} time steps in one launch)",
                    "bound": "hbm", "achieved": launch_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": launch_gbs / hbm_peak,
                    "traffic": traffic, "peak_source": peak_kind, "launches": 1, "avg_launch_ms": ms,
                    "algorithmic_bytes_per_launch": launch_bytes,
                    "persistent_kernel_phase_cycles_per_step": phase_cycles,
                    "per_kernel_path": per_kernel,
                    "note": "natural firing rates: about 0.7 MB of synapse rows per time step, so a step is bound by "
                            "latency (grid barrier, dependent loads), not by HBM; roofline_saturated shows the same "
                            "delivery code with enough spikes to be bandwidth-relevant.  traffic: " + traffic_note}
    else:
        # a sharded model runs on the persistent kernel only: its presynaptic phase is timed with clock64
        pre_s = phase_cycles["cycles_presynaptic"] * probe_steps / sm_hz
        nat_bytes = pev * bpe + psp * ALGO_BYTES_PER_SPIKE
        nat_gbs = nat_bytes / pre_s / 1e9 if pre_s > 0 else 0.0
        roofline = {"kernel": "fusedStepKernel (presynaptic phase)", "bound": "hbm", "achieved": nat_gbs,
                    "peak": hbm_peak, "unit": "GB/s", "frac": nat_gbs / hbm_peak, "traffic": None,
                    "peak_source": peak_kind, "launches": probe_steps,
                    "persistent_kernel_phase_cycles_per_step": phase_cycles,
                    "note": "rank 0; phase time from clock64 inside the persistent kernel (no kernel boundary to put "
                            "CUDA events on)"}

    # ---- same kernel at saturation: a quarter of every population spikes in one step ----
    roofline_sat = None
    if not args.no_saturated and world == 1:
        rng = np.random.default_rng(99)
        sat_events = 0
        out_deg = {}
        for s in net.syns:
            rl = rt.array(f"{s.name}.row_length").astype(np.int64)
            out_deg[s.src] = out_deg.get(s.src, 0) + rl
        sat_spikes = 0
        for p in net.pops:
            ids = np.sort(rng.choice(p.n, size=p.n // 4, replace=False)).astype(np.uint32)
            rt.set_spike_list(p.name, ids)
            if p.name in out_deg:
                sat_events += int(out_deg[p.name][ids].sum())
            sat_spikes += len(ids)
        rt.set_option("count_events", 0)
        for _ in range(3):
            rt.update_synapses()
        rt.enable_timing(True)
        rt.reset_timers()
        reps = 10
        for _ in range(reps):
            rt.update_synapses()
        rt.synchronize()
        sat_s = rt.timer("presynaptic_update") / reps
        rt.enable_timing(False)
        sat_bytes = sat_events * bpe + sat_spikes * ALGO_BYTES_PER_SPIKE
        roofline_sat = {"kernel": "tiledDeliverKernel (with tiledDecideKernel before it and presynapticSparseKernel, left nothing, after)",
                        "bound": "hbm", "achieved": sat_bytes / sat_s / 1e9,
                        "peak": hbm_peak, "unit": "GB/s", "frac": sat_bytes / sat_s / 1e9 / hbm_peak,
                        "traffic": None, "peak_source": peak_kind, "events_per_launch": sat_events,
                        "algorithmic_bytes_per_launch": sat_bytes, "launch_ms": sat_s * 1e3,
                        "events_per_s": sat_events / sat_s,
                        "note": "25% of every population spiking in one step; inputs larger than L2"}

    # ---- CPU baseline on this box's host (rank 0, N=1 only) ------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            # a bounded sample of the same architecture: about ten seconds of CPU time
            r = run_reference_sample(args.cpu_sample_scale, block, args.cpu_sample_blocks, 0)
            cpu = {"value": r["events_per_s"], "unit": "synaptic events/s", "cores": 1, "kind": r["kind"],
                   "realtime_factor": r["rtf"],
                   "sample": f"Potjans neuron_scale={args.cpu_sample_scale} (published in-degrees, {r['synapses']} synapses), "
                             f"{r['total_steps']} time steps, {r['seconds']:.2f} s of CPU time"}
        except Exception as e:      # the baseline is reported, never required
            cpu = {"value": None, "unit": "synaptic events/s", "cores": 1, "kind": "port", "sample": f"failed: {e}"}

    if rank == 0:
        n_neurons = sum(p.n for p in net.pops)
        line = {
            "metric": "synaptic events/s (Potjans microcircuit architecture)",
            "value": value, "unit": "synaptic events/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "realtime_factor": sim_seconds / seconds,
            "us_per_timestep": ms * 1e3 / (args.steps * block),
            "config": {"workload": f"Potjans-Diesmann microcircuit architecture x{scale:g}: {n_neurons} LIF neurons, "
                                   f"published in-degrees, SPARSE with dendritic delays, PoissonExp background, "
                                   f"dt=0.1 ms; one bench step = {block} time steps ({block * 1e-4:g} s biological)",
                       "parallelism": f"postsynaptic sharding over {world} GPU(s)" if world > 1 else "single GPU",
                       "schedule": ["persistent kernel, every synapse delivered before the neuron update",
                                    "persistent kernel, split delivery: synapses that arrive in the same step before the "
                                    "neuron update, all others behind it in the shadow of the second grid barrier",
                                    "persistent kernel, spikes delivered one step late (no synapse arrives in the same "
                                    "step): one grid barrier per step",
                                    "warp-specialised persistent kernel: synapses with a delay of 0 or 1 step delivered by "
                                    "the spiking thread inside the neuron update, all others streamed by dedicated warps "
                                    "over the next two steps; one grid barrier per step"][rt.schedule],
                       "min_delay_ms": args.min_delay,
                       "l2": "working set (2.5 GB of synapses) exceeds L2; no flush needed",
                       "spikes_per_s_biological": spikes / sim_seconds,
                       "mean_rates_hz": rates, "bytes_per_event": bpe},
            "clocks": clocks,
            "e2e": {"value": e2e_events / e2e_seconds, "unit": "synaptic events/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": d2h_moved, "recording_bytes_per_step": d2h,
                    "realtime_factor": sim_seconds / e2e_seconds,
                    "note": "GeNNModel.step_time + pull_recording_buffers_from_device into page-locked memory (the "
                            "recording's non-zero bit words travel as (index, word) pairs listed on the device; "
                            "recording_bytes_per_step is the size of the recording itself); "
                            "the model takes no per-step host input (background drive is drawn on the device, as in "
                            "the reference script)"},
            "gpu_launches": int(l1 - l0),
            "roofline": roofline,
            "roofline_saturated": roofline_sat,
            "cpu_baseline": cpu,
        }
    model.unload()
    # ---- parity: population statistics over --parity-seconds against the reference's ----------
    parity = None
    if args.parity_seconds > 0:
        parity = parity_leg(rank, world, local_rank, block, args.parity_seconds,
                            (lambda t: dist.all_reduce(t)) if world > 1 else None)
    if rank == 0:
        line["parity"] = parity
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
