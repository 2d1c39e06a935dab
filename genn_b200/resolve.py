"""Resolve a :class:`genn_b200.model.GeNNModel` description into flat arrays.

The resolved network is plain data in the reference's own memory layout
(ragged ELL rows with ``rowStride = maxRowLength`` for SPARSE, 32-bit words
with MSB-first bit order for BITMASK, row-major ``numPre x numPost`` for DENSE:
runtime.cc:336-402, presynapticUpdateStrategySIMT.cc:274-282).  It is what the
CUDA runtime uploads, and what :func:`write_netspec` serialises for tools that
read the text format.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

from .model import (GeNNModel, NeuronGroup, SynapseGroup, VarInit, _f32)


@dataclass
class RPop:
    name: str
    n: int
    kind: str
    params: Dict[str, float]
    derived: Dict[str, float]
    vars: Dict[str, np.ndarray]             # (batch, n); None when initialised on device
    var_inits: Dict[str, Optional[VarInit]]
    egps: Dict[str, np.ndarray]
    num_delay_slots: int = 1
    record: bool = False
    spike_time_required: bool = False


@dataclass
class RCurrentSource:
    name: str
    pop: str
    kind: str
    params: Dict[str, float]
    derived: Dict[str, float]
    vars: Dict[str, np.ndarray]


@dataclass
class RPsm:
    """One postsynaptic input buffer (``outPost`` [+ ``denDelay`` ring]); shared
    by every synapse group fused into it."""
    name: str
    trg: str
    kind: str
    params: Dict[str, float]
    derived: Dict[str, float]
    max_den_delay: int                      # 0: no dendritic delay ring
    members: List[str] = field(default_factory=list)


@dataclass
class RSyn:
    name: str
    matrix: str
    src: str
    trg: str
    wum: str
    wum_params: Dict[str, float]
    psm: int                                # index into Net.psms
    ax_delay: int
    back_delay: int
    max_den_delay: int
    row_stride: int
    ind_dtype: object
    row_length: Optional[np.ndarray] = None  # uint32 [numPre]
    ind: Optional[np.ndarray] = None         # uint32 [numPre*row_stride] (narrowed on upload)
    g: Optional[np.ndarray] = None           # float32, same indexing (or numPre*numPost for DENSE)
    d: Optional[np.ndarray] = None           # uint8
    gp: Optional[np.ndarray] = None          # uint32 words for BITMASK
    connect: object = None                   # SparseConnectInit when built on device
    var_inits: Dict[str, Optional[VarInit]] = field(default_factory=dict)
    procedural: bool = False
    num_threads_per_spike: int = 1


@dataclass
class Net:
    name: str
    dt: float
    seed: int
    batch_size: int
    fuse_psm: bool
    narrow_ind: bool
    pops: List[RPop]
    css: List[RCurrentSource]
    psms: List[RPsm]
    syns: List[RSyn]

    def pop(self, name: str) -> RPop:
        return next(p for p in self.pops if p.name == name)

    def syn(self, name: str) -> RSyn:
        return next(s for s in self.syns if s.name == name)


def _resolve_var(init, shape, dtype):
    """Host-resolvable initialisers become arrays; snippets stay symbolic."""
    if isinstance(init, VarInit):
        if init.snippet == "Constant":
            return np.full(shape, init.params["constant"], dtype=dtype), None
        return None, init
    arr = np.asarray(init, dtype=dtype)
    if arr.ndim == 0:
        return np.full(shape, arr, dtype=dtype), None
    return np.ascontiguousarray(np.broadcast_to(arr, shape)).astype(dtype), None


def ragged_from_pairs(pre: np.ndarray, post: np.ndarray, num_pre: int, per_syn: Dict[str, np.ndarray],
                      row_stride: Optional[int] = None):
    """(pre, post) pairs sorted by (pre, post) -> ragged rows.  Per-synapse
    arrays must already be in that order."""
    row_length = np.bincount(pre, minlength=num_pre).astype(np.uint32)
    stride = int(row_stride if row_stride is not None else max(1, row_length.max() if num_pre else 1))
    starts = np.zeros(num_pre + 1, dtype=np.int64)
    np.cumsum(row_length, out=starts[1:])
    col = np.arange(len(pre), dtype=np.int64) - starts[pre]
    flat = pre.astype(np.int64) * stride + col
    ind = np.zeros(num_pre * stride, dtype=np.uint32)
    ind[flat] = post
    out = {}
    for k, v in per_syn.items():
        a = np.zeros(num_pre * stride, dtype=v.dtype)
        a[flat] = v
        out[k] = a
    return row_length, stride, ind, out


def bitmask_from_pairs(pre: np.ndarray, post: np.ndarray, num_pre: int, num_post: int) -> np.ndarray:
    """Word-packed connectivity: bit ``gid = pre*stride + post`` with the row
    stride padded to 32 and bits counted from the MSB of each word
    (single_threaded_cpu/backend.cc:2003-2006)."""
    stride = ((num_post + 31) // 32) * 32
    gid = pre.astype(np.int64) * stride + post.astype(np.int64)
    words = np.zeros((num_pre * stride) // 32, dtype=np.uint32)
    np.bitwise_or.at(words, gid // 32, (np.uint32(0x80000000) >> (gid % 32).astype(np.uint32)))
    return words


def calc_max_row_length(snippet: str, params: Dict[str, float], num_pre: int, num_post: int) -> int:
    """Row stride for device-built connectivity: the 0.9999 quantile (over the
    whole matrix) of the row-length distribution, as the snippets'
    SET_CALC_MAX_ROW_LENGTH_FUNC do (initSparseConnectivitySnippet.h:130-160,
    338-346, 393-403), with a small safety margin because a row longer than
    the stride is an error here rather than a silent truncation."""
    from scipy.stats import binom
    q = 0.9999 ** (1.0 / num_pre)
    if snippet in ("FixedProbability", "FixedProbabilityNoAutapse"):
        n = binom.ppf(q, num_post, params["prob"])
    elif snippet == "FixedNumberTotalWithReplacement":
        n = binom.ppf(q, int(params["num"]), 1.0 / num_pre)
    elif snippet == "FixedNumberPreWithReplacement":
        n = binom.ppf(q, int(params["num"]) * num_post, 1.0 / num_pre)
    elif snippet == "FixedNumberPostWithReplacement":
        return int(params["num"])
    else:
        raise ValueError(snippet)
    return int(n) + 8


def resolve(model: GeNNModel) -> Net:
    dt = float(model.dt)
    batch = int(model.batch_size)
    pops: List[RPop] = []
    for p in model.neuron_populations.values():
        vars_, inits = {}, {}
        for name, var in p.vars.items():
            a, sn = _resolve_var(var.init, (batch, p.num_neurons), var.dtype)
            vars_[name], inits[name] = a, sn
        # a population needs as many spike slots as its longest outgoing axonal
        # delay plus one (neuronGroup.cc:408-411)
        slots = 1 + max([sg.axonal_delay_steps for sg in p.out_syn] +
                        [sg.back_prop_delay_steps for sg in p.in_syn] + [0])
        st_req = any(sg.has_learning for sg in p.out_syn) or any(sg.has_learning for sg in p.in_syn)
        pops.append(RPop(p.name, p.num_neurons, p.neuron_model, dict(p.params), p.derived_params(dt),
                         vars_, inits, {k: np.asarray(v) for k, v in p.extra_global_params.items()},
                         num_delay_slots=slots, record=bool(p.spike_recording_enabled),
                         spike_time_required=st_req))
    css = []
    for c in model.current_sources.values():
        vars_ = {}
        for name, var in c.vars.items():
            a, sn = _resolve_var(var.init, (batch, c.pop.num_neurons), var.dtype)
            if a is None:
                raise ValueError("current source variables must be host-initialised")
            vars_[name] = a
        css.append(RCurrentSource(c.name, c.pop.name, c.model_name, dict(c.params), c.derived_params(dt), vars_))

    psms: List[RPsm] = []
    psm_index: Dict[object, int] = {}
    syns: List[RSyn] = []
    for sg in model.synapse_populations.values():
        key = sg.psm_fuse_key() if model.fuse_postsynaptic_models else ("__own__", sg.name)
        if key not in psm_index:
            psm_index[key] = len(psms)
            psms.append(RPsm(sg.name, sg.trg.name, sg.ps.snippet, dict(sg.ps.params), sg.psm_derived_params(dt),
                             sg.max_dendritic_delay_timesteps if sg.has_dendritic_delay else 0))
        psms[psm_index[key]].members.append(sg.name)

        wum = {"StaticPulse": "STATIC", "StaticPulseConstantWeight": "CONST",
               "StaticPulseDendriticDelay": "DENDELAY", "STDP": "STDP"}[sg.wu.snippet]
        matrix = sg.matrix_type
        r = RSyn(sg.name, matrix, sg.src.name, sg.trg.name, wum, dict(sg.wu.params), psm_index[key],
                 sg.axonal_delay_steps, sg.back_prop_delay_steps,
                 sg.max_dendritic_delay_timesteps if sg.has_dendritic_delay else 0,
                 0, sg.ind_dtype, connect=sg.connect,
                 procedural=(matrix in ("PROCEDURAL", "DENSE_PROCEDURALG")),
                 num_threads_per_spike=sg.num_threads_per_spike)
        num_pre, num_post = sg.src.num_neurons, sg.trg.num_neurons
        per_syn, inits = {}, {}
        n_syn = None
        if sg._pre is not None:
            n_syn = len(sg._pre)
        for name, init in sg.wu.vars.items():
            dtype = np.uint8 if name == "d" else np.float32
            if isinstance(init, VarInit) and init.snippet != "Constant":
                inits[name] = init
            elif matrix in ("SPARSE", "BITMASK") and sg._pre is not None:
                arr = np.asarray(init.params["constant"] if isinstance(init, VarInit) else init, dtype=dtype)
                if arr.ndim == 0:
                    arr = np.full(n_syn, arr, dtype=dtype)
                elif len(arr) != n_syn:
                    raise ValueError(f"{sg.name}.{name}: {len(arr)} values for {n_syn} synapses")
                elif sg._order is not None:
                    arr = arr[sg._order]
                per_syn[name] = arr
            elif matrix == "DENSE":
                arr = np.asarray(init.params["constant"] if isinstance(init, VarInit) else init, dtype=dtype)
                per_syn[name] = (np.full(num_pre * num_post, arr, dtype=dtype) if arr.ndim == 0
                                 else np.ascontiguousarray(arr.reshape(num_pre * num_post)))
            else:
                inits[name] = init if isinstance(init, VarInit) else VarInit("Constant", {"constant": float(init)})
        r.var_inits = inits
        if matrix == "SPARSE":
            if sg._pre is not None:
                rl, stride, ind, out = ragged_from_pairs(sg._pre, sg._post, num_pre, per_syn, sg.max_connections)
                r.row_length, r.row_stride, r.ind = rl, stride, ind
                r.g, r.d = out.get("g"), out.get("d")
            else:
                r.row_stride = int(sg.max_connections or
                                   calc_max_row_length(sg.connect.snippet, sg.connect.params, num_pre, num_post))
            if getattr(sg, "trg_range", None) is not None:
                r.trg_range = sg.trg_range
        elif matrix == "BITMASK":
            r.row_stride = ((num_post + 31) // 32) * 32
            if sg._pre is not None:
                r.gp = bitmask_from_pairs(sg._pre, sg._post, num_pre, num_post)
        elif matrix == "DENSE":
            r.row_stride = num_post
            r.g = per_syn.get("g")
        else:
            # PROCEDURAL: nothing is stored, but rows are regenerated exactly as the initialisation
            # kernel would have written them, row stride (longest row) included
            if sg.connect is None:
                raise ValueError(f"{sg.name}: procedural connectivity needs a connectivity initialiser")
            r.row_stride = int(sg.max_connections or
                               calc_max_row_length(sg.connect.snippet, sg.connect.params, num_pre, num_post))
        syns.append(r)
    return Net(model.name, dt, int(model.seed), batch, bool(model.fuse_postsynaptic_models),
               bool(model.default_narrow_sparse_ind_enabled), pops, css, psms, syns)


# ---------------------------------------------------------------------------
# Text serialisation (one item per line, arrays as raw little-endian files)
# ---------------------------------------------------------------------------
def write_netspec(net: Net, directory: str, steps: int, dump_every: int = 0) -> str:
    """Write ``net`` as ``<directory>/spec.txt`` plus raw array files; returns
    the spec path.  Batch size must be 1 and every array host-resolved."""
    if net.batch_size != 1:
        raise ValueError("the text format describes batch size 1 only")
    os.makedirs(directory, exist_ok=True)

    def dump(name, arr):
        np.ascontiguousarray(arr).tofile(os.path.join(directory, name))
        return name

    lines = [f"name {net.name}", f"dt {net.dt!r}", f"seed {net.seed}", f"steps {steps}",
             f"dump_every {dump_every}", f"fuse_psm {int(net.fuse_psm)}", f"narrow_ind {int(net.narrow_ind)}"]
    for p in net.pops:
        if p.kind == "LIF":
            ps = " ".join(repr(float(p.params[k])) for k in ("C", "TauM", "Vrest", "Vreset", "Vthresh", "Ioffset", "TauRefrac"))
            lines.append(f"pop {p.name} {p.n} LIF {ps} " + dump(f"V_{p.name}.bin", p.vars["V"][0]) + " " +
                         dump(f"RefracTime_{p.name}.bin", p.vars["RefracTime"][0]))
        elif p.kind == "Izhikevich":
            ps = " ".join(repr(float(p.params[k])) for k in ("a", "b", "c", "d"))
            lines.append(f"pop {p.name} {p.n} IZH {ps} " + dump(f"V_{p.name}.bin", p.vars["V"][0]) + " " +
                         dump(f"U_{p.name}.bin", p.vars["U"][0]))
        elif p.kind == "SpikeSourceArray":
            lines.append(f"pop {p.name} {p.n} SSA " + dump(f"start_{p.name}.bin", p.vars["startSpike"][0]) + " " +
                         dump(f"end_{p.name}.bin", p.vars["endSpike"][0]) + " " +
                         dump(f"times_{p.name}.bin", p.egps["spikeTimes"].astype(np.float32)))
        elif p.kind == "Poisson":
            lines.append(f"pop {p.name} {p.n} POISSON {float(p.params['rate'])!r}")
        else:
            raise ValueError(p.kind)
    for c in net.css:
        if c.kind == "PoissonExp":
            lines.append(f"cs {c.name} {c.pop} POISSONEXP {float(c.params['weight'])!r} "
                         f"{float(c.params['tauSyn'])!r} {float(c.params['rate'])!r}")
        else:
            lines.append(f"cs {c.name} {c.pop} DC {float(c.params['amp'])!r}")
    for s in net.syns:
        psm = net.psms[s.psm]
        if s.matrix not in ("SPARSE", "BITMASK", "DENSE"):
            raise ValueError("procedural connectivity has no text form")
        item = [f"syn {s.name} {s.matrix} {s.src} {s.trg} wum {s.wum}"]
        if s.wum == "CONST":
            item.append(repr(float(s.wum_params["g"])))
        elif s.wum == "STDP":
            item += [repr(float(s.wum_params[k])) for k in ("tauPlus", "tauMinus", "Aplus", "Aminus", "Wmin", "Wmax")]
        item.append("psm " + {"ExpCurr": "EXPCURR", "ExpCond": "EXPCOND", "DeltaCurr": "DELTA"}[psm.kind])
        if psm.kind == "ExpCurr":
            item.append(repr(float(psm.params["tau"])))
        elif psm.kind == "ExpCond":
            item += [repr(float(psm.params["tau"])), repr(float(psm.params["E"]))]
        if s.ax_delay:
            item.append(f"axdelay {s.ax_delay}")
        if s.back_delay:
            item.append(f"backdelay {s.back_delay}")
        if s.max_den_delay:
            item.append(f"maxdendelay {s.max_den_delay}")
        if s.matrix == "SPARSE":
            item.append(f"maxconn {s.row_stride}")
            item.append("rowlength " + dump(f"rowLength_{s.name}.bin", s.row_length))
            item.append("ind " + dump(f"ind_{s.name}.bin", s.ind.astype(np.uint32)))
        elif s.matrix == "BITMASK":
            item.append("gp " + dump(f"gp_{s.name}.bin", s.gp))
        if s.g is not None:
            item.append("g " + dump(f"g_{s.name}.bin", s.g.astype(np.float32)))
        if s.d is not None:
            item.append("d " + dump(f"d_{s.name}.bin", s.d.astype(np.uint8)))
        lines.append(" ".join(item))
    path = os.path.join(directory, "spec.txt")
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    return path
