"""Memory plan: every array a resolved network needs and the group descriptors
that point at them.

This is the counterpart of ``Runtime::allocate`` (runtime.cc:147-662), which
walks the model, calls ``BackendBase::createArray`` for each variable and then
pushes one struct per merged-group element.  The plan is independent of where
the arrays live: an ``ArrayFactory`` supplies the memory.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import abi
from .model import _f32
from .resolve import Net, RPop, RSyn

TIME_MIN = np.float32(-3.402823466e+38)     # initial spike time: -TIME_MAX (definitions.h)


def shard_bounds(n: int, world: int):
    """Boundaries of the contiguous slices of a population of ``n`` neurons owned
    by ``world`` processes: multiples of 32 (a warp writes one spike-recording
    word), the last one ``n``."""
    b = [((n * r) // world) & ~31 for r in range(world)]
    return b + [n]


class _View:
    """A window into an array handle (same memory, offset pointer)."""

    def __init__(self, parent, offset: int, nbytes: int):
        self.parent, self.offset, self.nbytes = parent, offset, nbytes
        self.ptr = parent.ptr + offset
        if hasattr(parent, "buf"):
            self.buf = parent.buf[offset:offset + nbytes]


class ArrayFactory:
    """Where arrays live.  ``alloc`` returns a handle with an integer ``ptr``."""

    def alloc(self, nbytes: int):
        raise NotImplementedError

    def alloc_exchange(self, nbytes: int):
        """Memory that peers of a sharded model can map (spike lists and flags)."""
        return self.alloc(nbytes)

    def push(self, handle, host: np.ndarray):
        raise NotImplementedError

    def pull(self, handle, host: np.ndarray):
        raise NotImplementedError

    def memset(self, handle, value: int, nbytes: int):
        raise NotImplementedError


@dataclass
class PlannedArray:
    name: str
    handle: object
    dtype: np.dtype
    shape: Tuple[int, ...]

    @property
    def ptr(self) -> int:
        return self.handle.ptr

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize


@dataclass
class InitTask:
    """Work for the initialisation kernels (backendSIMT.cc:1368-1779)."""
    kind: str                   # "var" | "connect" | "sparse_var" | "remap"
    target: str                 # array name (or synapse group name)
    snippet: int = 0
    params: Tuple[float, ...] = ()
    stream: int = 0
    extra: Optional[dict] = None


class Plan:
    def __init__(self, net: Net, factory: ArrayFactory, num_recording_timesteps: Optional[int] = None,
                 shard: Optional[Tuple[int, int]] = None):
        self.net = net
        self.factory = factory
        self.num_recording_timesteps = int(num_recording_timesteps or 0)
        self.shard = shard
        self.arrays: Dict[str, PlannedArray] = {}
        self.init_tasks: List[InitTask] = []
        self.neuron_descs: List[abi.NeuronGroupDesc] = []
        self.synapse_descs: List[abi.SynapseGroupDesc] = []
        self._next_stream = 1
        self.exchange = None                # arena of a sharded model
        self.flags_offset = 0
        self._build()

    # ------------------------------------------------------------------
    def _stream(self) -> int:
        s = self._next_stream
        self._next_stream += 1
        return s

    def _new(self, name: str, dtype, shape, init=None) -> PlannedArray:
        dtype = np.dtype(dtype)
        shape = tuple(int(x) for x in shape)
        nbytes = max(1, int(np.prod(shape, dtype=np.int64))) * dtype.itemsize
        handle = self.factory.alloc(nbytes)
        arr = PlannedArray(name, handle, dtype, shape)
        self.arrays[name] = arr
        if init is None:
            self.factory.memset(handle, 0, nbytes)
        elif isinstance(init, np.ndarray):
            host = np.ascontiguousarray(init.astype(dtype, copy=False)).reshape(shape)
            self.factory.push(handle, host)
        else:
            self.factory.push(handle, np.full(shape, init, dtype=dtype))
        return arr

    def host_copy(self, name: str) -> np.ndarray:
        a = self.arrays[name]
        out = np.empty(a.shape, dtype=a.dtype)
        self.factory.pull(a.handle, out)
        return out

    def push(self, name: str, host: np.ndarray):
        a = self.arrays[name]
        self.factory.push(a.handle, np.ascontiguousarray(host.astype(a.dtype, copy=False)).reshape(a.shape))

    # ------------------------------------------------------------------
    def _build(self):
        net, B = self.net, self.net.batch_size
        pop_index = {p.name: i for i, p in enumerate(net.pops)}

        # a sharded model keeps every population's spike lists (one section per
        # process) and the arrival flags in ONE arena that peers can map
        world = self.shard[1] if self.shard else 1
        for p in net.pops:
            p.runtime_slots = p.num_delay_slots + 3     # three spare slots: see include/genn_b200.h
            bounds = shard_bounds(p.n, world)
            p.shard_bounds = bounds
            p.list_capacity = p.n if world == 1 else max(32, max(bounds[r + 1] - bounds[r] for r in range(world)))
        if world > 1:
            offset = 256
            layout = {}
            for p in net.pops:
                for name, nbytes in ((f"{p.name}.spk_cnt", world * B * p.runtime_slots * 4),
                                     (f"{p.name}.spk_tag", world * B * p.runtime_slots * 8),
                                     (f"{p.name}.spk_wire", world * B * p.runtime_slots * p.list_capacity * 8),
                                     (f"{p.name}.spk", world * B * p.runtime_slots * p.list_capacity * 4)):
                    layout[name] = (offset, nbytes)
                    offset = (offset + nbytes + 255) & ~255
            # the dendritic-delay rings too: the process that owns a spiking neuron may reduce its
            # nearest synapses straight into the rings of the process that owns the targets
            for i, psm in enumerate(net.psms):
                if psm.max_den_delay:
                    nbytes = B * psm.max_den_delay * net.pop(psm.trg).n * 4
                    layout[f"psm{i}.den_delay"] = (offset, nbytes)
                    offset = (offset + nbytes + 255) & ~255
            self.exchange = self.factory.alloc_exchange(offset)
            self.factory.memset(self.exchange, 0, offset)
            self._exchange_layout = layout

        # neuron-side arrays
        for p in net.pops:
            slots = p.runtime_slots
            for v, arr in p.vars.items():
                dtype = np.uint32 if p.kind == "SpikeSourceArray" else np.float32
                a = self._new(f"{p.name}.{v}", dtype, (B, p.n), arr if arr is not None else 0)
                if arr is None:
                    init = p.var_inits[v]
                    self.init_tasks.append(InitTask("var", a.name, abi.INIT_KINDS[init.snippet],
                                                    self._init_params(init), self._stream()))
            if p.kind == "SpikeSourceArray":
                times = p.egps.get("spikeTimes", np.zeros(1, np.float32)).astype(np.float32)
                if len(times) == 0:
                    times = np.zeros(1, np.float32)
                self._new(f"{p.name}.spikeTimes", np.float32, times.shape, times)
            if world == 1:
                self._new(f"{p.name}.spk_cnt", np.uint32, (B, slots))
                self._new(f"{p.name}.spk", np.uint32, (B, slots, p.n))
            else:
                for name, shape, dtype in ((f"{p.name}.spk_cnt", (world, B, slots), np.uint32),
                                           (f"{p.name}.spk_tag", (world, B, slots), np.uint64),
                                           (f"{p.name}.spk_wire", (world, B, slots, p.list_capacity), np.uint64),
                                           (f"{p.name}.spk", (world, B, slots, p.list_capacity), np.uint32)):
                    off, nbytes = self._exchange_layout[name]
                    self.arrays[name] = PlannedArray(name, _View(self.exchange, off, nbytes), np.dtype(dtype), shape)
            if p.spike_time_required:
                self._new(f"{p.name}.sT", np.float32, (B, slots, p.n), TIME_MIN)
            if p.record and self.num_recording_timesteps:
                # a process records the slice it updates
                lo, hi = (p.shard_bounds[self.shard[0]], p.shard_bounds[self.shard[0] + 1]) if self.shard else (0, p.n)
                self._new(f"{p.name}.record", np.uint32, (self.num_recording_timesteps, B, (hi - lo + 31) // 32))
        for c in net.css:
            for v, arr in c.vars.items():
                self._new(f"{c.name}.{v}", np.float32, (B, net.pop(c.pop).n), arr)

        # postsynaptic input buffers
        for i, psm in enumerate(net.psms):
            n = net.pop(psm.trg).n
            self._new(f"psm{i}.out_post", np.float32, (B, n))
            if psm.max_den_delay and world > 1:
                off, nbytes = self._exchange_layout[f"psm{i}.den_delay"]
                self.arrays[f"psm{i}.den_delay"] = PlannedArray(f"psm{i}.den_delay", _View(self.exchange, off, nbytes),
                                                                np.dtype(np.float32), (B, psm.max_den_delay, n))
            elif psm.max_den_delay:
                self._new(f"psm{i}.den_delay", np.float32, (B, psm.max_den_delay, n))

        # synapse-side arrays
        for s in net.syns:
            self._plan_synapse_arrays(s)

        # descriptors
        for p in net.pops:
            self.neuron_descs.append(self._neuron_desc(p))
        for s in net.syns:
            self.synapse_descs.append(self._synapse_desc(s))

    @staticmethod
    def _init_params(init) -> Tuple[float, ...]:
        from .model import VAR_INIT_SNIPPETS
        return tuple(float(init.params[k]) for k in VAR_INIT_SNIPPETS[init.snippet])

    def _plan_synapse_arrays(self, s: RSyn):
        net, B = self.net, self.net.batch_size
        ns, nt = net.pop(s.src).n, net.pop(s.trg).n
        learn = (s.wum == "STDP")
        gB = B if learn else 1
        if s.matrix == "SPARSE":
            stride = s.row_stride
            self._new(f"{s.name}.row_length", np.uint32, (ns,), s.row_length)
            self._new(f"{s.name}.ind", s.ind_dtype, (ns * stride,),
                      s.ind.astype(s.ind_dtype) if s.ind is not None else None)
            if s.ind is None:
                cp = tuple(float(v) for v in s.connect.params.values())
                self.init_tasks.append(InitTask("connect", s.name, abi.CONNECT_KINDS[s.connect.snippet], cp,
                                                self._stream(), {"num_src": ns, "num_trg": nt}))
            for v, dtype in (("g", np.float32), ("d", np.uint8)):
                have = getattr(s, v)
                if have is not None:
                    host = np.broadcast_to(have, (gB if v == "g" else 1, ns * stride))
                    self._new(f"{s.name}.{v}", dtype, host.shape, np.ascontiguousarray(host))
                elif v in s.var_inits:
                    init = s.var_inits[v]
                    a = self._new(f"{s.name}.{v}", dtype, (gB if v == "g" else 1, ns * stride))
                    params = self._init_params(init)
                    if init.snippet == "NormalClippedDelay":
                        params = tuple(x / net.dt for x in params)
                    self.init_tasks.append(InitTask("sparse_var", a.name, abi.INIT_KINDS[init.snippet], params,
                                                    self._stream(), {"syn": s.name}))
            if learn:
                if s.ind is None:
                    raise ValueError("learning synapse groups need host-supplied connectivity")
                cols = np.bincount(s.ind.reshape(ns, stride)[np.arange(stride)[None, :] < s.row_length[:, None]],
                                   minlength=nt)
                s.col_stride = int(max(1, cols.max()))
                self._new(f"{s.name}.col_length", np.uint32, (nt,))
                self._new(f"{s.name}.remap", np.uint32, (nt * s.col_stride,))
                self.init_tasks.append(InitTask("remap", s.name))
        elif s.procedural:
            # nothing to allocate: two Philox streams, the ones a SPARSE twin's initialisation would use
            s.proc_streams = (self._stream(), self._stream() if s.wum == "STATIC" else 0)
        elif s.matrix == "BITMASK":
            words = (ns * s.row_stride) // 32
            self._new(f"{s.name}.gp", np.uint32, (words,), s.gp)
        elif s.matrix == "DENSE":
            if s.g is not None:
                host = np.broadcast_to(s.g, (gB, ns * nt))
                self._new(f"{s.name}.g", np.float32, host.shape, np.ascontiguousarray(host))
            elif "g" in s.var_inits:
                init = s.var_inits["g"]
                a = self._new(f"{s.name}.g", np.float32, (gB, ns * nt))
                self.init_tasks.append(InitTask("var", a.name, abi.INIT_KINDS[init.snippet],
                                                self._init_params(init), self._stream()))

    def _ptr(self, name: str) -> Optional[int]:
        a = self.arrays.get(name)
        return a.ptr if a is not None else None

    def _neuron_desc(self, p: RPop) -> abi.NeuronGroupDesc:
        net = self.net
        d = abi.NeuronGroupDesc()
        d.model = abi.NEURON_KINDS[p.kind]
        d.num_neurons = p.n
        d.num_delay_slots = p.runtime_slots
        d.rng_stream = self._stream()
        if self.shard is not None:
            rank, world = self.shard
            d.first_neuron, d.num_update = p.shard_bounds[rank], p.shard_bounds[rank + 1] - p.shard_bounds[rank]
            d.spk_slot_stride = p.list_capacity
        else:
            d.first_neuron, d.num_update = 0, p.n
        if p.kind == "LIF":
            vals = [p.params["Vthresh"], p.params["Vreset"], p.params["Vrest"], p.params["Ioffset"],
                    p.derived["Rmembrane"], p.derived["ExpTC"], p.params["TauRefrac"]]
            names = ["V", "RefracTime"]
        elif p.kind == "Izhikevich":
            vals = [p.params[k] for k in "abcd"]
            names = ["V", "U"]
        elif p.kind == "SpikeSourceArray":
            vals, names = [], ["startSpike", "endSpike"]
            d.egp = self._ptr(f"{p.name}.spikeTimes")
        else:
            vals, names = [p.derived["isi"]], ["timeStepToSpike"]
        for i, v in enumerate(vals):
            d.params[i] = _f32(v)
        for i, v in enumerate(names):
            d.vars[i] = self._ptr(f"{p.name}.{v}")
        d.spk_cnt = self._ptr(f"{p.name}.spk_cnt")
        d.spk = self._ptr(f"{p.name}.spk")
        if self.shard is not None:          # this process writes its own section
            rank = self.shard[0]
            d.spk_cnt += rank * net.batch_size * p.runtime_slots * 4
            d.spk += rank * net.batch_size * p.runtime_slots * p.list_capacity * 4
            d.spk_tag = self._ptr(f"{p.name}.spk_tag") + rank * net.batch_size * p.runtime_slots * 8
            d.spk_wire = (self._ptr(f"{p.name}.spk_wire") +
                          rank * net.batch_size * p.runtime_slots * p.list_capacity * 8)
        d.spike_times = self._ptr(f"{p.name}.sT")
        d.record_spk = self._ptr(f"{p.name}.record")
        k = 0
        for i, psm in enumerate(net.psms):
            if psm.trg != p.name:
                continue
            if k >= abi.MAX_PSM:
                raise ValueError(f"population '{p.name}' has more than {abi.MAX_PSM} postsynaptic input buffers; "
                                 "enable fuse_postsynaptic_models")
            q = d.psm[k]
            q.model = abi.PSM_KINDS[psm.kind]
            q.max_den_delay = psm.max_den_delay
            if psm.kind == "ExpCurr":
                q.params[0], q.params[1] = _f32(psm.derived["init"]), _f32(psm.derived["expDecay"])
            elif psm.kind == "ExpCond":
                q.params[0], q.params[1] = _f32(psm.derived["expDecay"]), _f32(psm.params["E"])
            q.out_post = self._ptr(f"psm{i}.out_post")
            q.den_delay = self._ptr(f"psm{i}.den_delay")
            k += 1
        d.num_psm = k
        k = 0
        for c in net.css:
            if c.pop != p.name:
                continue
            if k >= abi.MAX_CS:
                raise ValueError(f"population '{p.name}' has more than {abi.MAX_CS} current sources")
            q = d.cs[k]
            q.model = abi.CS_KINDS[c.kind]
            q.rng_stream = self._stream()
            if c.kind == "DC":
                q.params[0] = _f32(c.params["amp"])
            else:
                q.params[0] = _f32(c.derived["Init"])
                q.params[1] = _f32(c.derived["ExpDecay"])
                q.params[2] = _f32(c.derived["ExpMinusLambda"])
                q.params[3] = _f32((c.params["rate"] / 1000.0) * net.dt)      # lambda
                q.var0 = self._ptr(f"{c.name}.current")
            k += 1
        d.num_cs = k
        return d

    def _synapse_desc(self, s: RSyn) -> abi.SynapseGroupDesc:
        net = self.net
        src, trg = net.pop(s.src), net.pop(s.trg)
        d = abi.SynapseGroupDesc()
        d.connectivity = abi.CONN_KINDS["PROCEDURAL" if s.procedural else s.matrix]
        d.wu_model = abi.WU_KINDS[s.wum]
        d.num_src, d.num_trg = src.n, trg.n
        d.row_stride = s.row_stride
        d.ind_bytes = np.dtype(s.ind_dtype).itemsize
        d.axonal_delay, d.back_prop_delay = s.ax_delay, s.back_delay
        d.src_delay_slots, d.trg_delay_slots = src.runtime_slots, trg.runtime_slots
        d.max_den_delay = s.max_den_delay
        d.col_stride = getattr(s, "col_stride", 0)
        if s.wum == "CONST":
            d.wu_params[0] = _f32(s.wum_params["g"])
        elif s.wum == "STDP":
            for i, k in enumerate(("tauPlus", "tauMinus", "Aplus", "Aminus", "Wmin", "Wmax")):
                d.wu_params[i] = _f32(s.wum_params[k])
            # spike times as seen at the synapse: sT + (delay + 1) * dt
            # (synapseUpdateGroupMerged.cc:118-142)
            d.wu_params[6] = _f32(net.dt * (s.ax_delay + 1))
            d.wu_params[7] = _f32(net.dt * (s.back_delay + 1))
        for f in ("row_length", "ind", "g", "d", "gp", "col_length", "remap"):
            setattr(d, f, self._ptr(f"{s.name}.{f}"))
        d.src_spk_cnt, d.src_spk = self._ptr(f"{src.name}.spk_cnt"), self._ptr(f"{src.name}.spk")
        if self.shard is not None:
            d.src_sections = self.shard[1]
            d.src_spk_slot_stride = src.list_capacity
            d.src_cnt_section_stride = net.batch_size * src.runtime_slots
            d.src_spk_section_stride = net.batch_size * src.runtime_slots * src.list_capacity
            d.src_spk_tag = self._ptr(f"{src.name}.spk_tag")
            d.src_spk_wire = self._ptr(f"{src.name}.spk_wire")
        d.trg_spk_cnt, d.trg_spk = self._ptr(f"{trg.name}.spk_cnt"), self._ptr(f"{trg.name}.spk")
        d.src_spike_times = self._ptr(f"{src.name}.sT")
        d.trg_spike_times = self._ptr(f"{trg.name}.sT")
        d.out_post = self._ptr(f"psm{s.psm}.out_post")
        d.den_delay = self._ptr(f"psm{s.psm}.den_delay")
        d.rng_stream = self._stream()
        if s.procedural:
            import math
            if s.wum not in ("STATIC", "CONST"):
                raise ValueError(f"{s.name}: procedural connectivity supports StaticPulse and StaticPulseConstantWeight")
            d.proc_connect = abi.CONNECT_KINDS[s.connect.snippet]
            cp = [float(v) for v in s.connect.params.values()] + [0.0] * 4
            if s.connect.snippet in ("FixedProbability", "FixedProbabilityNoAutapse"):
                cp[1] = 1.0 / math.log(1.0 - cp[0])
                cp[2] = float(s.num_threads_per_spike)      # sub-rows of a row, each with a stream of its own
            for i in range(4):
                d.proc_connect_params[i] = _f32(cp[i])
            d.rng_stream, d.proc_weight_stream = s.proc_streams
            if s.wum == "STATIC":
                init = s.var_inits["g"]
                d.proc_weight_init = abi.INIT_KINDS[init.snippet]
                for i, v in enumerate(self._init_params(init)):
                    d.proc_weight_params[i] = _f32(v)
        return d
