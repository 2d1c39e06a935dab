"""Small, bounded workloads for profiling single kernels under ncu.

    python -m genn_b200.probes presyn --scale 0.5 --fraction 0.25 --reps 3

builds the Potjans architecture at ``--scale`` times the neurons (in-degree
and therefore row lengths unchanged), marks ``--fraction`` of every population
as having spiked, and launches the presynaptic update ``--reps`` times.  The
device holds about 2.6 GB x scale; one launch reads about
scale x fraction x 2.1 GB, so scale 0.5 / fraction 0.25 is twice the L2.
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def presyn(args):
    from . import workloads
    from .runtime import Runtime
    model = workloads.potjans(neuron_scale=args.scale, seed=1234)
    model.build()
    rt = Runtime(model, None)
    net = rt.net
    rng = np.random.default_rng(99)
    events = 0
    out_deg = {}
    for s in net.syns:
        rl = rt.array(f"{s.name}.row_length").astype(np.int64)
        out_deg[s.src] = out_deg.get(s.src, 0) + rl
    spikes = 0
    for p in net.pops:
        ids = np.sort(rng.choice(p.n, size=max(1, int(p.n * args.fraction)), replace=False)).astype(np.uint32)
        rt.set_spike_list(p.name, ids)
        events += int(out_deg[p.name][ids].sum()) if p.name in out_deg else 0
        spikes += len(ids)
    rt.set_option("spike_lanes", args.lanes)
    for _ in range(2):
        rt.update_synapses()
    rt.enable_timing(True)
    rt.reset_timers()
    for _ in range(args.reps):
        rt.update_synapses()
    rt.synchronize()
    sec = rt.timer("presynaptic_update") / args.reps
    print(json.dumps({"probe": "presyn", "scale": args.scale, "fraction": args.fraction, "lanes": args.lanes,
                      "events_per_launch": events, "spikes_per_launch": spikes, "launch_ms": sec * 1e3,
                      "events_per_s": events / sec, "GBps_at_7B": (events * 7 + spikes * 8) / sec / 1e9}))
    rt.close()


def phases(args):
    """Per-phase SM cycles of the persistent fused-step kernel at natural rates."""
    from . import workloads
    from .runtime import Runtime
    model = workloads.potjans(neuron_scale=args.scale, seed=1234, min_delay=args.min_delay,
                              extra_delay_slots=1 if args.min_delay > 0 else 0)
    model.build()
    rt = Runtime(model, None)
    rt.set_option("count_events", args.count_events)
    if args.blocks_per_sm:
        rt.set_option("fused_blocks_per_sm", args.blocks_per_sm)
    rt.set_option("use_owner", args.owner)
    rt.set_option("owner_item_lanes", args.item_lanes)
    rt.set_option("use_lag", args.lag)
    rt.set_option("use_split", args.split)
    rt.set_option("use_emit", args.emit)
    rt.set_option("stream_warps", args.stream_warps)
    rt.step_time(args.warm)
    rt.synchronize()
    rt.set_option("fused_profile", 1)
    names = ["cycles_presynaptic", "cycles_barrier_a", "cycles_neuron", "cycles_barrier_b"]
    before = [rt.counter(n) for n in names]
    ms = rt.step_time_timed(args.steps)
    after = [rt.counter(n) for n in names]
    out = {"probe": "phases", "scale": args.scale, "steps": args.steps, "us_per_step": ms * 1e3 / args.steps,
           "step_path": rt.step_path(), "lagging": rt.lagging, "schedule": rt.schedule, "stream_warps": rt.counter("stream_warps"),
           "probes_per_step": [rt.counter(f"probe{i}") / (args.steps + args.warm) for i in range(8)]}
    for n, a, b in zip(names, before, after):
        out[n + "_per_step"] = (b - a) / args.steps
    cta = rt.cta_cycles().astype(np.float64) / args.steps
    if len(cta):
        out["cta_presyn_header_median"] = float(np.median(rt.header_cycles.astype(np.float64) / args.steps))
        for j, n in enumerate(["presynaptic", "barrier_a", "neuron", "barrier_b"]):
            col = cta[:, j]
            out["cta_" + n] = {"min": col.min(), "median": float(np.median(col)), "max": col.max(),
                               "argmax": int(col.argmax())}
    if args.dump and len(cta):
        out["per_cta"] = [[round(float(x)) for x in row] for row in cta]
    print(json.dumps(out))
    rt.close()


def e2e(args):
    """Where the end-to-end step (launch of `block` time steps + recording pull) spends its time."""
    import time
    from . import workloads
    model = workloads.potjans(neuron_scale=args.scale, seed=1234, record=True)
    model.build()
    model.load(num_recording_timesteps=args.block)
    rt = model._runtime
    rt.set_option("count_events", args.count_events)
    rt.step_time(3 * args.block)
    rt.synchronize()
    kernel_ms, launch_s, sync_s, pull_s = [], [], [], []
    for _ in range(args.reps):
        kernel_ms.append(rt.step_time_timed(args.block))
    for _ in range(args.reps):
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
    one_launch = rt.step_time_timed(args.reps * args.block) / args.reps
    print(json.dumps({"probe": "e2e", "block": args.block, "kernel_ms_per_block_separate_launches": kernel_ms,
                      "kernel_ms_per_block_one_launch": one_launch, "launch_call_ms": [x * 1e3 for x in launch_s],
                      "wait_ms": [x * 1e3 for x in sync_s], "pull_ms": [x * 1e3 for x in pull_s]}))
    rt.close()


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("presyn")
    p.add_argument("--scale", type=float, default=0.5)
    p.add_argument("--fraction", type=float, default=0.25)
    p.add_argument("--reps", type=int, default=3)
    p.add_argument("--lanes", type=int, default=16)
    p.set_defaults(fn=presyn)
    p = sub.add_parser("phases")
    p.add_argument("--scale", type=float, default=1.0)
    p.add_argument("--steps", type=int, default=2000)
    p.add_argument("--warm", type=int, default=2000)
    p.add_argument("--count-events", type=int, default=0)
    p.add_argument("--blocks-per-sm", type=int, default=0)
    p.add_argument("--owner", type=int, default=0)
    p.add_argument("--lag", type=int, default=1, help="deliver spikes one step late where every delay allows it")
    p.add_argument("--split", type=int, default=1, help="deliver only same-step synapses before the neuron update")
    p.add_argument("--emit", type=int, default=1, help="near synapses delivered by the spiking thread, one barrier per step")
    p.add_argument("--stream-warps", type=int, default=-1, help="-1 auto, 0 one warp set, n warps per CTA that only stream")
    p.add_argument("--min-delay", type=float, default=0.0, help="lower clip of the delay distribution in ms")
    p.add_argument("--item-lanes", type=int, default=32)
    p.add_argument("--dump", action="store_true", help="print the per-CTA phase cycles")
    p.set_defaults(fn=phases)
    p = sub.add_parser("e2e")
    p.add_argument("--scale", type=float, default=1.0)
    p.add_argument("--block", type=int, default=1000)
    p.add_argument("--reps", type=int, default=4)
    p.add_argument("--count-events", type=int, default=1)
    p.set_defaults(fn=e2e)
    args = ap.parse_args()
    args.fn(args)


if __name__ == "__main__":
    main()
