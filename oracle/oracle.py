"""Python driver for the C restatement in oracle/genn_oracle.c.

TEST INFRASTRUCTURE ONLY.  Runs a resolved network (genn_b200.resolve.Net) on
the CPU checker using the same memory plan and group descriptors as the CUDA
runtime, with host arrays in place of device arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Dict, Optional

import numpy as np

from genn_b200 import abi
from genn_b200.plan import ArrayFactory, Plan
from genn_b200.resolve import Net

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libgenn_oracle.so")


def build(force: bool = False) -> str:
    """Compile the C restatement (IEEE-strict: no contraction, no fast-math)."""
    src = os.path.join(HERE, "genn_oracle.c")
    deps = [src, os.path.join(REPO, "include", "genn_b200.h"), os.path.join(REPO, "include", "genn_b200_rng.h")]
    if force or not os.path.exists(LIB) or any(os.path.getmtime(d) > os.path.getmtime(LIB) for d in deps):
        subprocess.check_call(["/usr/bin/gcc", "-O2", "-std=c99", "-fPIC", "-shared", "-ffp-contract=off",
                               "-fno-fast-math", "-I", os.path.join(REPO, "include"), "-o", LIB, src, "-lm"])
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        l = C.CDLL(build())
        l.oracle_create.argtypes = [C.c_double, C.c_uint64, C.c_uint32]
        l.oracle_create.restype = C.c_void_p
        l.oracle_destroy.argtypes = [C.c_void_p]
        l.oracle_push_neuron_group.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(abi.NeuronGroupDesc)]
        l.oracle_push_synapse_group.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(abi.SynapseGroupDesc)]
        l.oracle_push_custom_update.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(abi.CustomUpdateDesc)]
        l.oracle_step.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64]
        l.oracle_step.restype = None
        l.oracle_custom_update.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32]
        l.oracle_custom_update.restype = None
        l.oracle_timestep.argtypes = [C.c_void_p]
        l.oracle_timestep.restype = C.c_uint64
        l.oracle_steps_done.argtypes = [C.c_void_p]
        l.oracle_steps_done.restype = C.c_uint64
        l.oracle_synaptic_events.argtypes = [C.c_void_p]
        l.oracle_synaptic_events.restype = C.c_uint64
        l.oracle_set_timestep.argtypes = [C.c_void_p, C.c_uint64]
        l.oracle_build_remap.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                         C.c_uint32, C.c_void_p, C.c_void_p]
        l.oracle_build_remap.restype = None
        l.oracle_init_var.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32, C.POINTER(C.c_float),
                                      C.c_uint64, C.c_uint32]
        l.oracle_init_var.restype = None
        l.oracle_init_sparse_vars.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32,
                                              C.POINTER(C.c_float), C.c_uint64, C.c_uint32]
        l.oracle_init_sparse_vars.restype = None
        l.oracle_init_sparse_connectivity.argtypes = [C.c_uint32, C.POINTER(C.c_float), C.c_uint32, C.c_uint32,
                                                      C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                                                      C.c_uint64, C.c_uint32]
        l.oracle_init_sparse_connectivity.restype = C.c_int
        l.oracle_init_fixed_number_pre.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                                   C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32]
        l.oracle_init_fixed_number_pre.restype = C.c_int
        _lib = l
    return _lib


def _params(values):
    return (C.c_float * 4)(*(list(values) + [0.0] * 4)[:4])


def init_var(count: int, dtype, snippet: int, params, seed: int, stream: int) -> np.ndarray:
    out = np.zeros(count, dtype=dtype)
    lib().oracle_init_var(out.ctypes.data, out.dtype.itemsize, count, snippet, _params(params), seed, stream)
    return out


def init_sparse_vars(row_length: np.ndarray, row_stride: int, dtype, snippet: int, params, seed: int,
                     stream: int) -> np.ndarray:
    rl = np.ascontiguousarray(row_length, dtype=np.uint32)
    out = np.zeros(len(rl) * row_stride, dtype=dtype)
    lib().oracle_init_sparse_vars(rl.ctypes.data, len(rl), row_stride, out.ctypes.data, out.dtype.itemsize, snippet,
                                  _params(params), seed, stream)
    return out


def init_sparse_connectivity(snippet: int, params, num_src: int, row_stride: int, ind_dtype, trg_begin: int,
                             trg_end: int, seed: int, stream: int, row_length: Optional[np.ndarray] = None):
    """Returns (row_length, ind, overflow)."""
    rl = (np.zeros(num_src, dtype=np.uint32) if row_length is None
          else np.ascontiguousarray(row_length, dtype=np.uint32).copy())
    ind = np.zeros(num_src * row_stride, dtype=ind_dtype)
    if snippet == abi.CONNECT_FIXED_NUMBER_PRE:
        ov = lib().oracle_init_fixed_number_pre(int(params[0]), num_src, row_stride, ind.dtype.itemsize, trg_begin,
                                                trg_end, rl.ctypes.data, ind.ctypes.data, seed, stream)
    else:
        ov = lib().oracle_init_sparse_connectivity(snippet, _params(params), num_src, row_stride, ind.dtype.itemsize,
                                                   trg_begin, trg_end, rl.ctypes.data, ind.ctypes.data, seed, stream)
    return rl, ind, bool(ov)


class _HostHandle:
    def __init__(self, nbytes: int):
        self.buf = np.zeros(nbytes, dtype=np.uint8)
        self.ptr = self.buf.ctypes.data


class NumpyFactory(ArrayFactory):
    def alloc(self, nbytes: int):
        return _HostHandle(nbytes)

    def push(self, handle, host: np.ndarray):
        flat = np.ascontiguousarray(host).view(np.uint8).reshape(-1)
        handle.buf[:len(flat)] = flat

    def pull(self, handle, host: np.ndarray):
        host.view(np.uint8).reshape(-1)[:] = handle.buf[:host.nbytes]

    def memset(self, handle, value: int, nbytes: int):
        handle.buf[:nbytes] = value


class OracleRunner:
    """Steps a resolved network on the CPU checker."""

    def __init__(self, net: Net, num_recording_timesteps: Optional[int] = None, shard=None):
        self.net = net
        self.plan = Plan(net, NumpyFactory(), num_recording_timesteps, shard=shard)
        for task in self.plan.init_tasks:
            if task.kind == "remap":
                self._build_remap(task.target)
            else:
                raise ValueError(f"the CPU checker takes host-initialised networks only ({task.kind}: {task.target})")
        self._l = lib()
        self._h = self._l.oracle_create(net.dt, net.seed, net.batch_size)
        for i, d in enumerate(self.plan.neuron_descs):
            self._l.oracle_push_neuron_group(self._h, i, C.byref(d))
        for i, d in enumerate(self.plan.synapse_descs):
            self._l.oracle_push_synapse_group(self._h, i, C.byref(d))
        self.num_recording_timesteps = int(num_recording_timesteps or 0)

    def _build_remap(self, syn_name: str):
        s = self.net.syn(syn_name)
        a = self.plan.arrays
        lib().oracle_build_remap(a[f"{syn_name}.row_length"].ptr, a[f"{syn_name}.ind"].ptr,
                                 np.dtype(s.ind_dtype).itemsize, self.net.pop(s.src).n, self.net.pop(s.trg).n,
                                 s.row_stride, s.col_stride, a[f"{syn_name}.col_length"].ptr,
                                 a[f"{syn_name}.remap"].ptr)

    def step(self, n: int = 1):
        self._l.oracle_step(self._h, n, self.num_recording_timesteps)

    def add_custom_update(self, operation: str, source: str, broadcast: bool = False, scale: float = 1.0) -> str:
        """Batch-reduce `source` ([batch, ...] fp32 array of the plan); returns the target array's name."""
        src = self.plan.arrays[source]
        elements = int(np.prod(src.shape[1:], dtype=np.int64))
        idx = getattr(self, "_num_custom", 0)
        trg = self.plan._new(f"cu.{idx}.reduction", np.float32, (elements,))
        d = abi.CustomUpdateDesc()
        d.op = abi.REDUCE_SUM if operation == "SUM" else abi.REDUCE_MAX
        d.broadcast, d.scale, d.num_elements = int(broadcast), scale, elements
        d.source, d.target = src.ptr, trg.ptr
        self._l.oracle_push_custom_update(self._h, idx, C.byref(d))
        self._num_custom = idx + 1
        return trg.name

    def custom_update(self):
        self._l.oracle_custom_update(self._h, 0, getattr(self, "_num_custom", 0))

    @property
    def timestep(self) -> int:
        return self._l.oracle_timestep(self._h)

    @property
    def synaptic_events(self) -> int:
        return self._l.oracle_synaptic_events(self._h)

    def array(self, name: str) -> np.ndarray:
        return self.plan.host_copy(name)

    def current_spikes(self, pop: str, batch: int = 0) -> np.ndarray:
        p = self.net.pop(pop)
        slots = p.runtime_slots
        slot = self._l.oracle_steps_done(self._h) % slots
        cnt = self.array(f"{pop}.spk_cnt")[batch, slot]
        return self.array(f"{pop}.spk")[batch, slot, :cnt].copy()

    def close(self):
        if self._h:
            self._l.oracle_destroy(self._h)
            self._h = None
