"""Host-side model description mirroring PyGeNN's ``GeNNModel`` API.

The names, argument meaning and error behaviour follow the reference's Python
front-end (pygenn/genn_model.py:179-847, pygenn/genn_groups.py) for the subset
of built-in models the B200 kernels implement, so a script written against
PyGeNN's ``add_neuron_population`` / ``add_synapse_population`` / ``build`` /
``load`` / ``step_time`` runs unchanged apart from the import.

This module is pure description: it owns no device memory and launches
nothing.  ``GeNNModel.load`` hands the description to :mod:`genn_b200.runtime`,
which drives the CUDA library through its C ABI.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import numpy as np

# ---------------------------------------------------------------------------
# Built-in model tables (names and parameter order as in the reference:
# neuronModels.h:163-325, postsynapticModels.h:93-151,
# currentSourceModels.h:60-129, weightUpdateModels.h:236-368)
# ---------------------------------------------------------------------------
NEURON_MODELS = {
    "LIF": dict(params=["C", "TauM", "Vrest", "Vreset", "Vthresh", "Ioffset", "TauRefrac"],
                vars=[("V", np.float32), ("RefracTime", np.float32)]),
    "Izhikevich": dict(params=["a", "b", "c", "d"],
                       vars=[("V", np.float32), ("U", np.float32)]),
    "SpikeSourceArray": dict(params=[],
                             vars=[("startSpike", np.uint32), ("endSpike", np.uint32)],
                             egps=["spikeTimes"]),
    "Poisson": dict(params=["rate"], vars=[("timeStepToSpike", np.float32)]),
}
POSTSYNAPTIC_MODELS = {
    "ExpCurr": dict(params=["tau"]),
    "ExpCond": dict(params=["tau", "E"]),
    "DeltaCurr": dict(params=[]),
}
CURRENT_SOURCE_MODELS = {
    "DC": dict(params=["amp"], vars=[]),
    "PoissonExp": dict(params=["weight", "tauSyn", "rate"], vars=[("current", np.float32)]),
}
WEIGHT_UPDATE_MODELS = {
    "StaticPulse": dict(params=[], vars=[("g", np.float32)]),
    "StaticPulseConstantWeight": dict(params=["g"], vars=[]),
    "StaticPulseDendriticDelay": dict(params=[], vars=[("g", np.float32), ("d", np.uint8)]),
    "STDP": dict(params=["tauPlus", "tauMinus", "Aplus", "Aminus", "Wmin", "Wmax"],
                 vars=[("g", np.float32)]),
}
VAR_INIT_SNIPPETS = {
    "Constant": ["constant"],
    "Uniform": ["min", "max"],
    "Normal": ["mean", "sd"],
    "NormalClipped": ["mean", "sd", "min", "max"],
    "NormalClippedDelay": ["mean", "sd", "min", "max"],
}
SPARSE_CONNECT_SNIPPETS = {
    "FixedProbability": ["prob"],
    "FixedProbabilityNoAutapse": ["prob"],
    "FixedNumberTotalWithReplacement": ["num"],
    "FixedNumberPreWithReplacement": ["num"],
    "FixedNumberPostWithReplacement": ["num"],
    "OneToOne": [],
}
MATRIX_TYPES = ("SPARSE", "BITMASK", "DENSE", "PROCEDURAL", "DENSE_PROCEDURALG")


def _f32(x) -> float:
    """Round a double to fp32, as the reference's code generator does when it
    prints derived parameters as ``float`` literals (type.cc:299-345)."""
    return float(np.float32(x))


@dataclass
class VarInit:
    """Initialiser for a state variable (pygenn ``init_var``)."""
    snippet: str
    params: Dict[str, float]


@dataclass
class SparseConnectInit:
    snippet: str
    params: Dict[str, float]


@dataclass
class PostsynapticInit:
    snippet: str
    params: Dict[str, float]
    vars: Dict[str, object] = field(default_factory=dict)
    var_refs: Dict[str, object] = field(default_factory=dict)


@dataclass
class WeightUpdateInit:
    snippet: str
    params: Dict[str, float]
    vars: Dict[str, object] = field(default_factory=dict)
    pre_vars: Dict[str, object] = field(default_factory=dict)
    post_vars: Dict[str, object] = field(default_factory=dict)


def init_var(snippet: str, params: Dict[str, float] = {}) -> VarInit:
    """pygenn.init_var (genn_model.py:849-871)."""
    if snippet not in VAR_INIT_SNIPPETS:
        raise ValueError(f"unsupported variable initialisation snippet '{snippet}'")
    missing = [p for p in VAR_INIT_SNIPPETS[snippet] if p not in params]
    if missing:
        raise ValueError(f"{snippet}: missing parameters {missing}")
    return VarInit(snippet, dict(params))


def init_sparse_connectivity(snippet: str, params: Dict[str, float] = {}) -> SparseConnectInit:
    """pygenn.init_sparse_connectivity (genn_model.py:873-895)."""
    if snippet not in SPARSE_CONNECT_SNIPPETS:
        raise ValueError(f"unsupported sparse connectivity snippet '{snippet}'")
    missing = [p for p in SPARSE_CONNECT_SNIPPETS[snippet] if p not in params]
    if missing:
        raise ValueError(f"{snippet}: missing parameters {missing}")
    return SparseConnectInit(snippet, dict(params))


def init_postsynaptic(snippet: str, params: Dict[str, float] = {}, vars: Dict = {},
                      var_refs: Dict = {}) -> PostsynapticInit:
    """pygenn.init_postsynaptic (genn_model.py:897-935)."""
    if snippet not in POSTSYNAPTIC_MODELS:
        raise ValueError(f"unsupported postsynaptic model '{snippet}'")
    _check_params(snippet, POSTSYNAPTIC_MODELS[snippet]["params"], params)
    return PostsynapticInit(snippet, dict(params), dict(vars), dict(var_refs))


def init_weight_update(snippet: str, params: Dict[str, float] = {}, vars: Dict = {},
                       pre_vars: Dict = {}, post_vars: Dict = {}) -> WeightUpdateInit:
    """pygenn.init_weight_update (genn_model.py:937-985)."""
    if snippet not in WEIGHT_UPDATE_MODELS:
        raise ValueError(f"unsupported weight update model '{snippet}'")
    _check_params(snippet, WEIGHT_UPDATE_MODELS[snippet]["params"], params)
    want = [v for v, _ in WEIGHT_UPDATE_MODELS[snippet]["vars"]]
    if sorted(want) != sorted(vars.keys()):
        raise ValueError(f"{snippet}: variables {sorted(vars.keys())} given, {sorted(want)} expected")
    return WeightUpdateInit(snippet, dict(params), dict(vars), dict(pre_vars), dict(post_vars))


def _check_params(what: str, names: Sequence[str], params: Dict[str, float]):
    if sorted(names) != sorted(params.keys()):
        raise ValueError(f"{what}: parameters {sorted(params.keys())} given, {sorted(names)} expected")


class Variable:
    """A state variable: host view plus, once loaded, a device array.

    Mirrors pygenn's ``Variable`` (model_preprocessor.py:264-311): ``view`` is
    the host numpy array, ``push_to_device`` / ``pull_from_device`` copy it."""

    def __init__(self, name: str, dtype, init, shape):
        self.name = name
        self.dtype = np.dtype(dtype)
        self.init = init
        self.shape = tuple(shape)
        self._view: Optional[np.ndarray] = None
        self._array = None      # runtime.DeviceArray once loaded

    @property
    def view(self) -> np.ndarray:
        if self._view is None:
            if self._array is None:
                raise RuntimeError(f"variable '{self.name}' is not loaded")
            self._view = np.zeros(self.shape, dtype=self.dtype)     # host side made on first use
        return self._view

    @property
    def values(self) -> np.ndarray:
        return self.view.copy()

    @values.setter
    def values(self, v):
        self.view[...] = v

    def push_to_device(self):
        self._array.push(self.view)

    def pull_from_device(self):
        self._array.pull(self.view)

    @property
    def device_pointer(self) -> int:
        return self._array.ptr


class NeuronGroup:
    """A neuron population (pygenn ``NeuronGroupMixin``, genn_groups.py:233-330)."""

    def __init__(self, model: "GeNNModel", name: str, num_neurons: int, neuron: str,
                 params: Dict[str, float], vars: Dict[str, object]):
        if neuron not in NEURON_MODELS:
            raise ValueError(f"unsupported neuron model '{neuron}'")
        spec = NEURON_MODELS[neuron]
        _check_params(neuron, spec["params"], params)
        want = [v for v, _ in spec["vars"]]
        if sorted(want) != sorted(vars.keys()):
            raise ValueError(f"{neuron}: variables {sorted(vars.keys())} given, {sorted(want)} expected")
        self._model = model
        self.name = name
        self.num_neurons = int(num_neurons)
        self.neuron_model = neuron
        self.params = dict(params)
        self.vars: Dict[str, Variable] = {
            v: Variable(v, dt, vars[v], (model.batch_size, self.num_neurons)) for v, dt in spec["vars"]}
        self.extra_global_params: Dict[str, np.ndarray] = {}
        self.spike_recording_enabled = False
        self.current_sources: List["CurrentSource"] = []
        self.in_syn: List["SynapseGroup"] = []
        self.out_syn: List["SynapseGroup"] = []
        self._spike_recording_data = None
        # filled by load()
        self.num_delay_slots = 1

    # -- derived parameters (neuronModels.h:250-252, 322) ---------------------
    def derived_params(self, dt: float) -> Dict[str, float]:
        p = self.params
        if self.neuron_model == "LIF":
            return {"ExpTC": math.exp(-dt / p["TauM"]), "Rmembrane": p["TauM"] / p["C"]}
        if self.neuron_model == "Poisson":
            return {"isi": 1000.0 / (p["rate"] * dt)}
        return {}

    @property
    def spike_recording_data(self):
        """[(times, ids)] per batch, as pygenn (genn_groups.py:306-318)."""
        if self._spike_recording_data is None:
            raise RuntimeError("spike recording data has not been pulled")
        return self._spike_recording_data

    def set_extra_global_param(self, name: str, value):
        self.extra_global_params[name] = np.asarray(value)

    @property
    def current_spikes(self) -> np.ndarray:
        """Ids of the neurons that spiked in the last time step (batch 0)."""
        return self._model._runtime.current_spikes(self, 0)

    def get_current_spikes(self, batch: int = 0) -> np.ndarray:
        return self._model._runtime.current_spikes(self, batch)


class CurrentSource:
    def __init__(self, model: "GeNNModel", name: str, cs_model: str, pop: NeuronGroup,
                 params: Dict[str, float], vars: Dict[str, object]):
        if cs_model not in CURRENT_SOURCE_MODELS:
            raise ValueError(f"unsupported current source model '{cs_model}'")
        spec = CURRENT_SOURCE_MODELS[cs_model]
        _check_params(cs_model, spec["params"], params)
        self.name = name
        self.model_name = cs_model
        self.pop = pop
        self.params = dict(params)
        self.vars: Dict[str, Variable] = {
            v: Variable(v, dt, vars.get(v, 0.0), (model.batch_size, pop.num_neurons)) for v, dt in spec["vars"]}

    def derived_params(self, dt: float) -> Dict[str, float]:
        p = self.params
        if self.model_name == "PoissonExp":   # currentSourceModels.h:125-128
            return {"ExpDecay": math.exp(-dt / p["tauSyn"]),
                    "Init": p["weight"] * (1.0 - math.exp(-dt / p["tauSyn"])) * (p["tauSyn"] / dt),
                    "ExpMinusLambda": math.exp(-(p["rate"] / 1000.0) * dt)}
        return {}


class SynapseGroup:
    """A synapse population (pygenn ``SynapseGroupMixin``, genn_groups.py:333-700)."""

    def __init__(self, model: "GeNNModel", name: str, matrix_type: str, src: NeuronGroup,
                 trg: NeuronGroup, wu: WeightUpdateInit, ps: PostsynapticInit,
                 connect: Optional[SparseConnectInit]):
        if matrix_type not in MATRIX_TYPES:
            raise ValueError(f"unsupported matrix type '{matrix_type}'")
        self._model = model
        self.name = name
        self.matrix_type = matrix_type
        self.src = src
        self.trg = trg
        self.wu = wu
        self.ps = ps
        self.connect = connect
        self.axonal_delay_steps = 0
        self.back_prop_delay_steps = 0
        self.max_dendritic_delay_timesteps = 1
        self.num_threads_per_spike = 1
        self.parallelism_hint = "POSTSYNAPTIC"
        self.narrow_sparse_ind_enabled = model.default_narrow_sparse_ind_enabled
        self.max_connections: Optional[int] = None
        self._pre = None
        self._post = None
        self._order = None
        self.vars: Dict[str, Variable] = {}
        self.out_post: Optional[Variable] = None
        # host copies of the ragged matrix once loaded
        self.row_lengths: Optional[np.ndarray] = None
        self.ind: Optional[np.ndarray] = None
        if matrix_type in ("SPARSE", "BITMASK") and connect is None:
            pass    # connectivity must be supplied with set_sparse_connections
        src.out_syn.append(self)
        trg.in_syn.append(self)

    @property
    def has_dendritic_delay(self) -> bool:
        return self.wu.snippet == "StaticPulseDendriticDelay"

    @property
    def has_learning(self) -> bool:
        return self.wu.snippet == "STDP"

    @property
    def weight_kind(self) -> str:
        return "CONSTANT" if self.wu.snippet == "StaticPulseConstantWeight" else "INDIVIDUAL"

    def set_sparse_connections(self, pre_indices, post_indices, presorted: bool = False):
        """Host-supplied connectivity (genn_groups.py:434-470): the pairs are
        sorted by (pre, post) and per-synapse variable arrays passed to
        ``init_weight_update`` are re-ordered the same way; multapses are kept.
        ``presorted``: the pairs already come row by row (non-decreasing presynaptic
        index) and are kept in the order given (no sort: large host-generated networks)."""
        if self.matrix_type not in ("SPARSE", "BITMASK"):
            raise Exception("set_sparse_connections only supports SPARSE and BITMASK format connectivity")
        pre = np.asarray(pre_indices, dtype=np.uint32)
        post = np.asarray(post_indices, dtype=np.uint32)
        if pre.shape != post.shape or pre.ndim != 1:
            raise Exception("pre and post synaptic index lists must be 1D arrays of the same length")
        if len(pre) and (pre.max() >= self.src.num_neurons or post.max() >= self.trg.num_neurons):
            raise Exception("synaptic indices out of range")
        if presorted:
            if len(pre) > 1 and np.any(pre[1:] < pre[:-1]):
                raise Exception("presorted connectivity must have non-decreasing presynaptic indices")
            order = None
            self._pre, self._post = pre, post
        else:
            order = np.lexsort((post, pre))
            self._pre = pre[order]
            self._post = post[order]
        self._order = order
        row_lengths = np.bincount(self._pre, minlength=self.src.num_neurons).astype(np.uint32)
        self.row_lengths = row_lengths
        if self.matrix_type == "SPARSE":
            longest = int(row_lengths.max()) if len(row_lengths) else 0
            self.max_connections = max(1, longest)

    @property
    def ind_dtype(self):
        """Narrowest index type that can address the target population when
        narrow indices are enabled (synapseGroup.cc:907-922)."""
        if self.narrow_sparse_ind_enabled:
            if self.trg.num_neurons <= 0xFF:
                return np.uint8
            if self.trg.num_neurons <= 0xFFFF:
                return np.uint16
        return np.uint32

    def psm_derived_params(self, dt: float) -> Dict[str, float]:
        p = self.ps.params
        if self.ps.snippet == "ExpCurr":    # postsynapticModels.h:104-106
            return {"expDecay": math.exp(-dt / p["tau"]),
                    "init": (p["tau"] * (1.0 - math.exp(-dt / p["tau"]))) * (1.0 / dt)}
        if self.ps.snippet == "ExpCond":
            return {"expDecay": math.exp(-dt / p["tau"])}
        return {}

    def psm_fuse_key(self):
        """Groups that share this key share one postsynaptic input buffer when
        ``fuse_postsynaptic_models`` is set (neuronGroup.cc:430-517)."""
        return (self.trg.name, self.ps.snippet, tuple(sorted(self.ps.params.items())),
                self.max_dendritic_delay_timesteps if self.has_dendritic_delay else 0,
                self.has_dendritic_delay)

    def pull_connectivity_from_device(self):
        self._model._runtime.pull_connectivity(self)

    def get_sparse_pre_inds(self) -> np.ndarray:
        rl = self.row_lengths
        return np.repeat(np.arange(self.src.num_neurons, dtype=np.uint32), rl)

    def get_sparse_post_inds(self) -> np.ndarray:
        stride = self.max_connections
        ind = self.ind.reshape(self.src.num_neurons, stride)
        mask = np.arange(stride)[None, :] < self.row_lengths[:, None]
        return ind[mask]


class CustomUpdate:
    """Batch-reduce custom update over per-synapse or per-neuron variables.

    Mirrors the reference's custom updates whose model reads a DUPLICATE
    variable and writes a REDUCE_BATCH_SUM / REDUCE_BATCH_MAX target
    (customUpdateModels.h, backendSIMT.cc:888-927, 1109-1147)."""

    def __init__(self, name: str, group_name: str, operation: str, source, target: str,
                 broadcast: bool = False, scale: float = 1.0):
        if operation not in ("SUM", "MAX"):
            raise ValueError("operation must be SUM or MAX")
        self.name = name
        self.group_name = group_name
        self.operation = operation
        self.source = source        # (SynapseGroup|NeuronGroup|CurrentSource, var name)
        self.target_name = target
        self.broadcast = bool(broadcast)    # write scale * reduced value back into every batch copy
        self.scale = float(scale)
        self.vars: Dict[str, Variable] = {}


class GeNNModel:
    """Mirror of ``pygenn.GeNNModel`` (genn_model.py:179-847) for the B200
    backend.  ``backend`` is accepted for source compatibility; there is one
    backend and no CPU fallback."""

    def __init__(self, precision: str = "float", model_name: str = "GeNNModel",
                 backend: Optional[str] = None, **preference_kwargs):
        if precision != "float":
            raise ValueError("the B200 backend computes in fp32 ('float') only")
        if backend not in (None, "b200"):
            raise KeyError(backend)
        self.precision = precision
        self.name = model_name
        self.dt = 1.0
        self.seed = 0
        self.batch_size = 1
        self.timing_enabled = False
        self.fuse_postsynaptic_models = False
        self.default_narrow_sparse_ind_enabled = False
        self.neuron_populations: Dict[str, NeuronGroup] = {}
        self.synapse_populations: Dict[str, SynapseGroup] = {}
        self.current_sources: Dict[str, CurrentSource] = {}
        self.custom_updates: Dict[str, CustomUpdate] = {}
        self.preferences = dict(preference_kwargs)
        self._built = False
        self._loaded = False
        self._runtime = None

    # -- PyGeNN spells the time step both ways ---------------------------------
    @property
    def dT(self):
        return self.dt

    @dT.setter
    def dT(self, v):
        self.dt = v

    @property
    def timestep(self) -> int:
        return self._runtime.timestep if self._runtime else 0

    @timestep.setter
    def timestep(self, v: int):
        self._runtime.timestep = int(v)

    @property
    def t(self) -> float:
        return self.timestep * self.dt

    def add_neuron_population(self, pop_name: str, num_neurons: int, neuron: str,
                              params: Dict[str, float] = {}, vars: Dict[str, object] = {}) -> NeuronGroup:
        if self._built:
            raise Exception("GeNN model already built")
        if pop_name in self.neuron_populations:
            raise ValueError(f"Neuron population '{pop_name}' already exists")
        pop = NeuronGroup(self, pop_name, num_neurons, neuron, params, vars)
        self.neuron_populations[pop_name] = pop
        return pop

    def add_synapse_population(self, pop_name: str, matrix_type: str, source: NeuronGroup,
                               target: NeuronGroup, weight_update_init: WeightUpdateInit,
                               postsynaptic_init: PostsynapticInit,
                               connectivity_init: Optional[SparseConnectInit] = None) -> SynapseGroup:
        if self._built:
            raise Exception("GeNN model already built")
        if pop_name in self.synapse_populations:
            raise ValueError(f"synapse population '{pop_name}' already exists")
        sg = SynapseGroup(self, pop_name, matrix_type, source, target, weight_update_init,
                          postsynaptic_init, connectivity_init)
        self.synapse_populations[pop_name] = sg
        return sg

    def add_current_source(self, cs_name: str, current_source_model: str, pop: NeuronGroup,
                           params: Dict[str, float] = {}, vars: Dict[str, object] = {}) -> CurrentSource:
        if self._built:
            raise Exception("GeNN model already built")
        if cs_name in self.current_sources:
            raise ValueError(f"current source '{cs_name}' already exists")
        cs = CurrentSource(self, cs_name, current_source_model, pop, params, vars)
        pop.current_sources.append(cs)
        self.current_sources[cs_name] = cs
        return cs

    def add_custom_update(self, cu_name: str, group_name: str, operation: str, source, target: str = "reduction",
                          broadcast: bool = False, scale: float = 1.0):
        if self._built:
            raise Exception("GeNN model already built")
        cu = CustomUpdate(cu_name, group_name, operation, source, target, broadcast, scale)
        self.custom_updates[cu_name] = cu
        return cu

    def build(self, path_to_model: str = "./", always_rebuild: bool = False, never_rebuild: bool = False):
        """Validate the description.  The kernels are precompiled sm_100a
        templates, so nothing is generated or compiled here; the call exists so
        PyGeNN scripts run unchanged (genn_model.py:649-706)."""
        if self._built:
            raise Exception("GeNN model already built")
        for sg in self.synapse_populations.values():
            if sg.matrix_type in ("SPARSE", "BITMASK") and sg._pre is None and sg.connect is None:
                raise Exception(f"synapse population '{sg.name}' has no connectivity")
            if sg.has_dendritic_delay and sg.max_dendritic_delay_timesteps < 1:
                raise Exception("max_dendritic_delay_timesteps must be at least 1")
        self._built = True

    def load(self, num_recording_timesteps: Optional[int] = None, **runtime_kwargs):
        if not self._built:
            raise Exception("GeNN model has to be built before running")
        if self._loaded:
            raise Exception("GeNN model already loaded")
        from .runtime import Runtime    # imports the CUDA library; fails loudly without it
        self._runtime = Runtime(self, num_recording_timesteps, **runtime_kwargs)
        self._loaded = True

    def unload(self):
        if self._runtime is not None:
            self._runtime.close()
        self._runtime = None
        self._loaded = False

    def step_time(self, num_steps: int = 1):
        """Advance the simulation (genn_model.py:817-822).  ``num_steps`` > 1
        replays the captured step graph back to back without returning to Python."""
        if not self._loaded:
            raise Exception("GeNN model has to be loaded before stepping")
        self._runtime.step_time(num_steps)

    def custom_update(self, name: str, all_reduce: bool = False):
        """Run custom update group ``name``.  ``all_reduce``: combine the reduced values of all processes
        of a data-parallel run (every process holds a share of the batch) before writing them back."""
        if not self._loaded:
            raise Exception("GeNN model has to be loaded before performing custom update")
        self._runtime.custom_update(name, all_reduce)

    def pull_recording_buffers_from_device(self):
        if not self._loaded:
            raise Exception("GeNN model has to be loaded before pulling recording buffers")
        self._runtime.pull_recording_buffers()

    @property
    def neuron_update_time(self) -> float:
        return self._runtime.timer("neuron_update")

    @property
    def presynaptic_update_time(self) -> float:
        return self._runtime.timer("presynaptic_update")

    @property
    def postsynaptic_update_time(self) -> float:
        return self._runtime.timer("postsynaptic_update")

    @property
    def init_time(self) -> float:
        return self._runtime.timer("init")

    @property
    def init_sparse_time(self) -> float:
        return self._runtime.timer("init_sparse")

    def get_custom_update_time(self, name: str) -> float:
        return self._runtime.timer("custom_update_" + name)
