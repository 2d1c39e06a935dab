"""Runtime: loads a model description onto the GPU and steps it through the
C ABI of the CUDA library.  Counterpart of ``GeNN::Runtime::Runtime``
(runtime.cc:147-718) for the B200 backend.  There is no CPU path: importing
this module without the built library raises.
"""
from __future__ import annotations

import ctypes as C
import os
import math
from typing import Dict, Optional, Tuple

import numpy as np

from . import abi
from .abi import check
from .plan import ArrayFactory, Plan
from .resolve import Net, resolve


class DeviceArray:
    def __init__(self, rt: "DeviceFactory", nbytes: int):
        self._rt = rt
        self.nbytes = nbytes
        p = C.c_void_p()
        check(rt.lib.b200_array_alloc(rt.handle, nbytes, C.byref(p)))
        self.ptr = p.value

    def push(self, host: np.ndarray):
        self._rt.push(self, host)

    def pull(self, host: np.ndarray):
        self._rt.pull(self, host)


class DeviceFactory(ArrayFactory):
    def __init__(self, lib, handle):
        self.lib = lib
        self.handle = handle
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def alloc(self, nbytes: int) -> DeviceArray:
        return DeviceArray(self, nbytes)

    def alloc_exchange(self, nbytes: int):
        p = C.c_void_p()
        check(self.lib.b200_exchange_alloc(self.handle, nbytes, C.byref(p)))
        arr = DeviceArray.__new__(DeviceArray)
        arr._rt, arr.nbytes, arr.ptr = self, nbytes, p.value
        return arr

    def push(self, handle: DeviceArray, host: np.ndarray):
        host = np.ascontiguousarray(host)
        check(self.lib.b200_array_push(self.handle, handle.ptr, host.ctypes.data, host.nbytes))
        self.h2d_bytes += host.nbytes

    def pull(self, handle: DeviceArray, host: np.ndarray):
        assert host.flags["C_CONTIGUOUS"]
        check(self.lib.b200_array_pull(self.handle, host.ctypes.data, handle.ptr, host.nbytes))
        self.d2h_bytes += host.nbytes

    def memset(self, handle: DeviceArray, value: int, nbytes: int):
        check(self.lib.b200_array_memset(self.handle, handle.ptr, value, nbytes))


def all_gather_bytes(payload: bytes):
    """All-gather a small byte string over the default ``torch.distributed`` group
    (any backend: this is bootstrap plumbing, not the data path)."""
    import torch.distributed as dist
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, payload)
    return out


class _LazyRecording:
    """List-like [(times, ids)] per batch element, decoded on first access."""

    def __init__(self, rt, pop):
        self._rt, self._pop, self._data = rt, pop, None

    def _get(self):
        if self._data is None:
            self._data = self._rt.recorded_spikes(self._pop)
        return self._data

    def __getitem__(self, i):
        return self._get()[i]

    def __len__(self):
        return len(self._get())

    def __iter__(self):
        return iter(self._get())


class Runtime:
    """One loaded model on one GPU."""

    def __init__(self, model, num_recording_timesteps: Optional[int] = None, device: int = 0,
                 shard: Optional[Tuple[int, int]] = None, net: Optional[Net] = None, exchange=None,
                 sharded_emit: Optional[bool] = None, local_peers=None):
        self.lib = abi.load_library()
        self.model = model
        self.device = int(device)
        self.net = net if net is not None else resolve(model)
        self.num_recording_timesteps = int(num_recording_timesteps or 0)
        h = C.c_void_p()
        check(self.lib.b200_runner_create(device, self.net.dt, self.net.seed, self.net.batch_size, C.byref(h)))
        self.handle = h
        self.factory = DeviceFactory(self.lib, self.handle)
        self._pinned = []
        self._rec_host = {}
        self.recording_pairs_capacity = None        # (index, word) pairs a recording pull has room for; None: 1/16 of the words
        self._rec_compact = None        # device pair list, device counter, their page-locked copies, capacity
        self._rec_pairs, self._rec_layout = None, {}
        self._rec_timestep = 0
        self.shard = shard
        # rank -> device pointer of a peer arena that is already addressable in this process
        self.local_peers = dict(local_peers or {})
        self.plan = Plan(self.net, self.factory, self.num_recording_timesteps, shard=shard)
        if shard is not None and shard[1] > 1:
            self._connect_peers(exchange)
        self._run_init_tasks()
        for i, d in enumerate(self.plan.neuron_descs):
            check(self.lib.b200_push_neuron_update_group(self.handle, i, C.byref(d)))
        for i, d in enumerate(self.plan.synapse_descs):
            check(self.lib.b200_push_synapse_group(self.handle, i, C.byref(d)))
        check(self.lib.b200_initialize(self.handle))
        check(self.lib.b200_initialize_sparse(self.handle))
        if shard is not None and shard[1] > 1:
            # delivering spikes one step late needs every process to do it: agree
            mine = bytes([1 if self.counter("lag_eligible") else 0])
            everyone = (exchange or all_gather_bytes)(mine)
            self.set_option("lag_agreed", 1.0 if all(b[0] for b in everyone) else 0.0)
            # "deliver at emission" across processes (near synapses travel through per-CTA queues) is the default
            # from 8 processes on, where it measured faster than the split schedule (13.1 against 14.4 us per
            # step of the Potjans x8 network); on 2 and 4 GPUs the split schedule is ahead (11.1 / 11.4 against
            # 12.2 / 11.9 us).  sharded_emit or GENN_B200_SHARDED_EMIT=0/1 (the same on every process) overrides.
            if sharded_emit is None:
                env = os.environ.get("GENN_B200_SHARDED_EMIT")
                sharded_emit = (env == "1") if env is not None else (shard[1] >= 8)
            if sharded_emit:
                self._exchange_near_tables(exchange or all_gather_bytes)
        self._cu_targets = {}
        if model is not None:
            self._bind_model_views()
            self._push_custom_updates()
            if getattr(model, "timing_enabled", False):
                check(self.lib.b200_enable_timing(self.handle, 1))
        self.synchronize()

    # -- sharded models: map every peer's exchange arena ---------------------------
    def _connect_peers(self, exchange):
        """``exchange(bytes) -> [bytes per rank]`` all-gathers the 64-byte IPC handle
        of this process's arena; the default uses ``torch.distributed``."""
        rank, world = self.shard
        handle = C.create_string_buffer(64)
        check(self.lib.b200_exchange_get_handle(self.handle, handle))
        handles = (exchange or all_gather_bytes)(handle.raw)
        if len(handles) != world:
            raise abi.B200Error(f"expected {world} arena handles, got {len(handles)}")
        for peer, h in enumerate(handles):
            if peer == rank:
                continue
            if peer in self.local_peers:
                # a pointer, or a callable that is given the arena size and returns one
                where = self.local_peers[peer]
                total = C.c_size_t(0)
                check(self.lib.b200_exchange_bytes(self.handle, C.byref(total)))
                where = where(total.value) if callable(where) else where
                check(self.lib.b200_exchange_set_peer(self.handle, peer, C.c_void_p(where)))
            else:
                check(self.lib.b200_exchange_open_peer(self.handle, peer, C.create_string_buffer(h, 64)))
        check(self.lib.b200_exchange_configure(self.handle, rank, world))

    def _exchange_near_tables(self, gather):
        """Sharded "deliver at emission" schedule: every process builds the nearest synapses (dendritic
        delay 0 or 1) of all source neurons onto its own neurons and hands every process the rows of
        that process's neurons (include/genn_b200.h: b200_near_export / import / finish)."""
        groups = len(self.plan.neuron_descs)
        handle = C.create_string_buffer(64)
        meta = (C.c_uint64 * (3 + 2 * groups))()
        check(self.lib.b200_near_export(self.handle, handle, meta, len(meta)))
        everyone = gather(handle.raw + bytes(meta))
        agreed = all(int.from_bytes(p[64:72], "little") == 1 for p in everyone)
        if agreed:
            metas = [(C.c_uint64 * (3 + 2 * groups)).from_buffer_copy(p[64:]) for p in everyone]
            # one row length per neuron group for all processes: the longest any of them needs
            common = (C.c_uint32 * groups)()
            for g in range(groups):
                shifts = [int(m[4 + 2 * g]) & 0xFFFFFFFF for m in metas]
                real = [x for x in shifts if x != 0xFFFFFFFF]
                common[g] = max(real) if len(real) == len(shifts) else 0xFFFFFFFF
            for peer, payload in enumerate(everyone):
                check(self.lib.b200_near_import(self.handle, peer, C.create_string_buffer(payload[:64], 64), metas[peer],
                                                common))
        gather(b"imported")          # nobody frees its table before everybody has copied from it
        check(self.lib.b200_near_finish(self.handle, int(agreed)))

    # -- initialisation kernels -------------------------------------------------
    def _run_init_tasks(self):
        a = self.plan.arrays
        for task in self.plan.init_tasks:
            params = (C.c_float * 4)(*(list(task.params) + [0.0] * 4)[:4])
            if task.kind == "var":
                arr = a[task.target]
                count = int(np.prod(arr.shape, dtype=np.int64))
                check(self.lib.b200_init_var(self.handle, arr.ptr, arr.dtype.itemsize, count, task.snippet,
                                             params, task.stream))
            elif task.kind == "connect":
                self._init_connectivity(task, params)
            elif task.kind == "sparse_var":
                s = self.net.syn(task.extra["syn"])
                arr = a[task.target]
                check(self.lib.b200_init_sparse_vars(self.handle, a[f"{s.name}.row_length"].ptr,
                                                     self.net.pop(s.src).n, s.row_stride, arr.ptr,
                                                     arr.dtype.itemsize, task.snippet, params, task.stream))
            elif task.kind == "remap":
                s = self.net.syn(task.target)
                check(self.lib.b200_build_remap(self.handle, a[f"{s.name}.row_length"].ptr, a[f"{s.name}.ind"].ptr,
                                                np.dtype(s.ind_dtype).itemsize, self.net.pop(s.src).n,
                                                self.net.pop(s.trg).n, s.row_stride, s.col_stride,
                                                a[f"{s.name}.col_length"].ptr, a[f"{s.name}.remap"].ptr))

    def _init_connectivity(self, task, params):
        s = self.net.syn(task.target)
        a = self.plan.arrays
        ns, nt = self.net.pop(s.src).n, self.net.pop(s.trg).n
        begin, end = getattr(s, "trg_range", (0, nt))
        snippet = task.snippet
        if snippet == abi.CONNECT_FIXED_NUMBER_TOTAL:
            # row lengths are drawn on the host from the multinomial, as the
            # reference's host initialisation code does
            # (initSparseConnectivitySnippet.h:300-336)
            rng = np.random.default_rng([self.net.seed, task.stream])
            rl = rng.multinomial(int(task.params[0]), np.full(ns, 1.0 / ns)).astype(np.uint32)
            if rl.max() > s.row_stride:
                raise abi.B200Error(f"{s.name}: drawn row length {rl.max()} exceeds max_connections {s.row_stride}")
            self.plan.push(f"{s.name}.row_length", rl)
        elif snippet in (abi.CONNECT_FIXED_PROBABILITY, abi.CONNECT_FIXED_PROBABILITY_NO_AUTAPSE):
            params[1] = 1.0 / math.log(1.0 - task.params[0])
            params[2] = float(s.num_threads_per_spike)      # sub-rows of a row (init.cuh: generateRow)
        check(self.lib.b200_init_sparse_connectivity(self.handle, snippet, params, ns, nt, s.row_stride,
                                                     np.dtype(s.ind_dtype).itemsize, begin, end,
                                                     a[f"{s.name}.row_length"].ptr, a[f"{s.name}.ind"].ptr,
                                                     task.stream))

    # -- PyGeNN-style views -----------------------------------------------------
    def _bind_model_views(self):
        m, a = self.model, self.plan.arrays
        for p in m.neuron_populations.values():
            for name, var in p.vars.items():
                arr = a[f"{p.name}.{name}"]
                var._array = arr.handle
                var.shape = arr.shape
        for c in m.current_sources.values():
            for name, var in c.vars.items():
                arr = a[f"{c.name}.{name}"]
                var._array = arr.handle
                var.shape = arr.shape
        from .model import Variable
        for sg in m.synapse_populations.values():
            rs = self.net.syn(sg.name)
            sg.max_connections = rs.row_stride if rs.matrix == "SPARSE" else sg.max_connections
            for name in ("g", "d"):
                arr = a.get(f"{sg.name}.{name}")
                if arr is not None:
                    v = Variable(name, arr.dtype, None, arr.shape)
                    v._array = arr.handle
                    sg.vars[name] = v
            arr = a[f"psm{rs.psm}.out_post"]
            v = Variable("outPost", arr.dtype, None, arr.shape)
            v._array = arr.handle
            sg.out_post = v
            if rs.matrix == "SPARSE" and rs.row_length is not None:
                sg.row_lengths, sg.ind = rs.row_length, rs.ind

    def pull_connectivity(self, sg):
        rs = self.net.syn(sg.name)
        sg.row_lengths = self.array(f"{sg.name}.row_length")
        sg.ind = self.array(f"{sg.name}.ind").astype(np.uint32)

    # -- stepping ---------------------------------------------------------------
    def step_time(self, num_steps: int = 1):
        check(self.lib.b200_step_time(self.handle, num_steps, self.num_recording_timesteps))

    def step_time_timed(self, num_steps: int) -> float:
        """Steps bracketed by CUDA events on the runner's stream; returns milliseconds."""
        ms = C.c_float()
        check(self.lib.b200_step_time_timed(self.handle, num_steps, self.num_recording_timesteps, C.byref(ms)))
        return float(ms.value)

    def timed_begin(self):
        """CUDA event on the runner's stream; ``timed_end`` returns the milliseconds since."""
        check(self.lib.b200_timed_begin(self.handle))

    def timed_end(self) -> float:
        ms = C.c_float()
        check(self.lib.b200_timed_end(self.handle, C.byref(ms)))
        return float(ms.value)

    def update_synapses(self):
        check(self.lib.b200_update_synapses(self.handle))

    def update_neurons(self):
        check(self.lib.b200_update_neurons(self.handle, self.num_recording_timesteps))

    def _push_custom_updates(self):
        """One batch-reduce descriptor per custom update of the model, merged by group name."""
        from .model import Variable
        per_group = {}
        for cu in self.model.custom_updates.values():
            obj, var = cu.source
            src = self.plan.arrays[f"{obj.name}.{var}"]
            if src.dtype != np.float32 or src.shape[0] != self.net.batch_size:
                raise abi.B200Error(f"custom update {cu.name}: {obj.name}.{var} is not a per-batch fp32 variable")
            elements = int(np.prod(src.shape[1:], dtype=np.int64))
            trg = self.plan._new(f"cu.{cu.name}.{cu.target_name}", np.float32, (elements,))
            d = abi.CustomUpdateDesc()
            d.op = abi.REDUCE_SUM if cu.operation == "SUM" else abi.REDUCE_MAX
            d.broadcast, d.scale, d.num_elements = int(cu.broadcast), cu.scale, elements
            d.source, d.target = src.ptr, trg.ptr
            idx = per_group.get(cu.group_name, 0)
            per_group[cu.group_name] = idx + 1
            check(self.lib.b200_push_custom_update(self.handle, cu.group_name.encode(), idx, C.byref(d)))
            self._cu_targets.setdefault(cu.group_name, []).append((trg, cu.operation))
            v = Variable(cu.target_name, np.float32, None, (elements,))
            v._array = trg.handle
            cu.vars[cu.target_name] = v

    def init_data_parallel(self, rank: Optional[int] = None, world: Optional[int] = None, gather=None):
        """Every process holds a share of the batch: create the NCCL communicator over which the batch-reduce
        custom updates combine their values (the reference: enableNCCLReductions and the three ncclXxx symbols
        of the generated library, genn_model.py / backends/cuda/backend.cc:219-226).  Rank 0 obtains the id;
        ``gather(bytes) -> [bytes per rank]`` hands it round (default: ``torch.distributed``)."""
        if rank is None or world is None:
            import torch.distributed as dist
            rank, world = dist.get_rank(), dist.get_world_size()
        ident = C.create_string_buffer(128)
        if rank == 0:
            check(self.lib.b200_nccl_unique_id(ident))
        everyone = (gather or all_gather_bytes)(ident.raw)
        if len(everyone) != world:
            raise abi.B200Error(f"expected {world} ids, got {len(everyone)}")
        check(self.lib.b200_nccl_init(self.handle, C.create_string_buffer(everyone[0], 128), rank, world))
        self.data_parallel = (rank, world)

    def custom_update(self, name: str, all_reduce: bool = False):
        """``all_reduce``: a data-parallel run: the reduced values are combined over all processes before
        they are written back (the communicator is created on first use if init_data_parallel was not called)."""
        if all_reduce and getattr(self, "data_parallel", None) is None:
            self.init_data_parallel()
        check(self.lib.b200_custom_update(self.handle, name.encode()))

    def synchronize(self):
        check(self.lib.b200_synchronize(self.handle))

    def set_option(self, name: str, value: float):
        check(self.lib.b200_set_option(self.handle, name.encode(), float(value)))

    @property
    def timestep(self) -> int:
        v = C.c_uint64()
        check(self.lib.b200_get_timestep(self.handle, C.byref(v)))
        return int(v.value)

    @timestep.setter
    def timestep(self, t: int):
        check(self.lib.b200_set_timestep(self.handle, int(t)))

    @property
    def steps_done(self) -> int:
        v = C.c_uint64()
        check(self.lib.b200_get_steps_done(self.handle, C.byref(v)))
        return int(v.value)

    def counter(self, name: str) -> int:
        v = C.c_uint64()
        check(self.lib.b200_get_counter(self.handle, name.encode(), C.byref(v)))
        return int(v.value)

    @property
    def kernel_launches(self) -> int:
        v = C.c_uint64()
        check(self.lib.b200_get_kernel_launches(self.handle, C.byref(v)))
        return int(v.value)

    def step_path(self):
        """(path, reason): 2 target-stationary persistent kernel, 1 persistent kernel with global
        reductions, 0 one launch per kernel; reason says why path 2 was not taken."""
        path = C.c_int()
        why = C.create_string_buffer(256)
        check(self.lib.b200_get_step_path(self.handle, C.byref(path), why, 256))
        return path.value, why.value.decode()

    @property
    def lagging(self) -> bool:
        """True if the persistent kernel delivers spikes one step late (every dendritic
        delay is at least one step), which lets it drop the second grid barrier."""
        return bool(self.counter("lag"))

    @property
    def schedule(self) -> int:
        """Schedule of the next persistent launch: 0 every synapse before the neuron update,
        1 only the synapses that arrive in the same step before it (split delivery),
        2 spikes delivered one step late (one grid barrier per step)."""
        return self.counter("schedule")

    def cta_cycles(self) -> np.ndarray:
        """[num_ctas, 4] cycles per phase of the persistent kernel (option fused_profile)."""
        out = np.zeros((1024, 4), dtype=np.uint64)
        n = C.c_uint32()
        check(self.lib.b200_get_cta_cycles(self.handle, out.ctypes.data, 1024, C.byref(n)))
        self.header_cycles = out.reshape(-1)[4 * n.value:5 * n.value].copy()
        return out[:n.value]

    def enable_timing(self, on: bool):
        check(self.lib.b200_enable_timing(self.handle, int(on)))

    def reset_timers(self):
        check(self.lib.b200_reset_timers(self.handle))

    def timer(self, name: str) -> float:
        v = C.c_double()
        check(self.lib.b200_get_timer(self.handle, name.encode(), C.byref(v)))
        return float(v.value)

    # -- data access --------------------------------------------------------------
    def array(self, name: str) -> np.ndarray:
        self.synchronize()
        return self.plan.host_copy(name)

    def current_spikes(self, pop, batch: int = 0) -> np.ndarray:
        name = pop if isinstance(pop, str) else pop.name
        p = self.net.pop(name)
        slot = self.steps_done % p.runtime_slots
        cnt, spk = self.array(f"{name}.spk_cnt"), self.array(f"{name}.spk")
        if cnt.ndim == 2:
            return spk[batch, slot, :int(cnt[batch, slot])].copy()
        # sharded: one section per process; a section's count travels in the low half
        # of its (step, count) word
        tag, wire = self.array(f"{name}.spk_tag"), self.array(f"{name}.spk_wire")
        out = []
        for s in range(tag.shape[0]):
            n = int(tag[s, batch, slot] & 0xFFFFFFFF)
            words = wire[s, batch, slot, :n]
            assert np.all((words >> 32) == (tag[s, batch, slot] >> 32)), "spike words of another step in the list"
            out.append((words & 0xFFFFFFFF).astype(np.uint32))
        return np.concatenate(out)

    def pinned_empty(self, shape, dtype) -> np.ndarray:
        """Page-locked host array (cudaHostAlloc) owned by this runtime."""
        dtype = np.dtype(dtype)
        nbytes = max(1, int(np.prod(shape, dtype=np.int64)) * dtype.itemsize)
        p = C.c_void_p()
        check(self.lib.b200_host_alloc(self.handle, nbytes, C.byref(p)))
        self._pinned.append(p.value)
        buf = (C.c_uint8 * nbytes).from_address(p.value)
        return np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape, dtype=np.int64))).reshape(shape)

    def pull_recording_buffers(self):
        """Bring the spike recording of the last ``num_recording_timesteps`` steps to page-locked host memory
        (Runtime::pullRecordingBuffersFromDevice, runtime.cc:720-746, copies the bit words whole).  A recording is
        almost all zeros at cortical rates, so the device first lists its non-zero words (b200_compact_words) and
        only (index, word) pairs travel; a recording too dense for the pair buffer is copied whole instead.
        Decoding into (times, ids) happens lazily in :meth:`recorded_spikes`."""
        T = self.num_recording_timesteps
        if not T:
            raise Exception("Recording buffer not allocated - cannot pull from device")
        self.synchronize()          # (reports device-side checks of the steps behind the recording)
        recs = [(p.name, self.plan.arrays[f"{p.name}.record"]) for p in self.net.pops if f"{p.name}.record" in self.plan.arrays]
        self._rec_pairs, self._rec_layout = None, {}
        total = sum(int(np.prod(a.shape, dtype=np.int64)) for _, a in recs)
        if recs and total < (1 << 32):
            if self._rec_compact is None:
                # room for one non-zero word in sixteen unless the caller chose
                cap = self.recording_pairs_capacity or max(1024, total // 16)
                self._rec_compact = (self.factory.alloc(cap * 8), self.factory.alloc(4), self.pinned_empty((cap, 2), np.uint32),
                                     self.pinned_empty((1,), np.uint32), cap)
            pairs, counter, host_pairs, host_count, cap = self._rec_compact
            check(self.lib.b200_array_memset(self.handle, counter.ptr, 0, 4))
            base = 0
            for name, arr in recs:
                n = int(np.prod(arr.shape, dtype=np.int64))
                check(self.lib.b200_compact_words(self.handle, arr.ptr, n, base, pairs.ptr, cap, counter.ptr))
                self._rec_layout[name] = (base, arr.shape)
                base += n
            check(self.lib.b200_array_pull(self.handle, host_count.ctypes.data, counter.ptr, 4))     # waits for the stream
            self.factory.d2h_bytes += 4
            count = int(host_count[0])
            if count <= cap:
                if count:
                    check(self.lib.b200_array_pull(self.handle, host_pairs.ctypes.data, pairs.ptr, count * 8))
                    self.factory.d2h_bytes += count * 8
                self._rec_pairs = host_pairs[:count].copy()
        self._rec_timestep = self.timestep
        for name, arr in recs:
            if self._rec_pairs is None:
                host = self._rec_host.get(name)
                if host is None:
                    host = self._rec_host[name] = self.pinned_empty(arr.shape, arr.dtype)
                self.factory.pull(arr.handle, host)
            if self.model is not None:
                self.model.neuron_populations[name]._spike_recording_data = _LazyRecording(self, name)

    def _recording_words(self, pop: str) -> np.ndarray:
        """The pulled recording of ``pop`` as its array of bit words [T][batch][words]."""
        if self._rec_pairs is None:
            return self._rec_host[pop]
        base, shape = self._rec_layout[pop]
        n = int(np.prod(shape, dtype=np.int64))
        words = np.zeros(n, dtype=np.uint32)
        idx = self._rec_pairs[:, 0].astype(np.int64) - base
        mine = (idx >= 0) & (idx < n)
        words[idx[mine]] = self._rec_pairs[mine, 1]
        return words.reshape(shape)

    def recorded_spikes(self, pop: str):
        """Decode pulled recording words into [(times, ids)] per batch element,
        as Runtime::getRecordedEvents does (runtime.cc:855-913)."""
        T = self.num_recording_timesteps
        ts = self._rec_timestep
        if ts < T:
            raise Exception("Event recording data can only be accessed once buffer is full")
        p = self.net.pop(pop)
        # a process of a sharded model records the slice of the population it updates
        lo, hi = (p.shard_bounds[self.shard[0]], p.shard_bounds[self.shard[0] + 1]) if self.shard else (0, p.n)
        start = (ts - T) * self.net.dt
        # the buffer is a ring over timestep % T: rotate so index 0 is the oldest step
        words = np.roll(self._recording_words(pop), -(ts % T), axis=0)
        out = []
        for b in range(self.net.batch_size):
            bits = np.unpackbits(np.ascontiguousarray(words[:, b, :]).view(np.uint8), axis=1, bitorder="little")
            step, ids = np.nonzero(bits[:, :hi - lo])
            out.append((start + step * self.net.dt, (ids + lo).astype(np.uint32)))
        return out

    # -- measurement helpers ------------------------------------------------------
    def set_spike_list(self, pop: str, ids: np.ndarray, batch: int = 0):
        """Overwrite the spike list the NEXT presynaptic update will read for
        ``pop`` (zero axonal delay).  Used to drive the presynaptic kernels with a
        chosen load when measuring them in isolation."""
        p = self.net.pop(pop)
        slot = self.steps_done % p.runtime_slots
        cnt = self.array(f"{pop}.spk_cnt")
        cnt[batch, slot] = len(ids)
        self.plan.push(f"{pop}.spk_cnt", cnt)
        arr = self.plan.arrays[f"{pop}.spk"]
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        offset = ((batch * p.runtime_slots + slot) * p.n) * 4
        check(self.lib.b200_array_push(self.handle, arr.ptr + offset, ids.ctypes.data, ids.nbytes))

    def close(self):
        if self.handle:
            for p in self._pinned:
                self.lib.b200_host_free(self.handle, p)
            self._pinned = []
            self.lib.b200_runner_destroy(self.handle)
            self.handle = None
