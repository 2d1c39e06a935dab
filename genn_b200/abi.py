"""ctypes mirror of include/genn_b200.h (descriptor structs, enums, prototypes)."""
from __future__ import annotations

import ctypes as C
import os

MAX_PSM, MAX_CS, MAX_PARAMS, MAX_VARS = 8, 4, 8, 4

NEURON_LIF, NEURON_IZHIKEVICH, NEURON_SPIKE_SOURCE_ARRAY, NEURON_POISSON = range(4)
PSM_EXP_CURR, PSM_EXP_COND, PSM_DELTA_CURR = range(3)
CS_DC, CS_POISSON_EXP = range(2)
WU_STATIC_PULSE, WU_CONSTANT_WEIGHT, WU_DENDRITIC_DELAY, WU_STDP = range(4)
CONN_SPARSE, CONN_BITMASK, CONN_DENSE, CONN_PROCEDURAL = range(4)
INIT_CONSTANT, INIT_UNIFORM, INIT_NORMAL, INIT_NORMAL_CLIPPED, INIT_NORMAL_CLIPPED_DELAY = range(5)
(CONNECT_FIXED_PROBABILITY, CONNECT_FIXED_PROBABILITY_NO_AUTAPSE, CONNECT_FIXED_NUMBER_TOTAL,
 CONNECT_FIXED_NUMBER_PRE, CONNECT_FIXED_NUMBER_POST) = range(5)
REDUCE_SUM, REDUCE_MAX = range(2)
OK, ERR_CUDA, ERR_INVALID, ERR_STATE, ERR_DEVICE_CHECK = range(5)

NEURON_KINDS = {"LIF": NEURON_LIF, "Izhikevich": NEURON_IZHIKEVICH,
                "SpikeSourceArray": NEURON_SPIKE_SOURCE_ARRAY, "Poisson": NEURON_POISSON}
PSM_KINDS = {"ExpCurr": PSM_EXP_CURR, "ExpCond": PSM_EXP_COND, "DeltaCurr": PSM_DELTA_CURR}
CS_KINDS = {"DC": CS_DC, "PoissonExp": CS_POISSON_EXP}
WU_KINDS = {"STATIC": WU_STATIC_PULSE, "CONST": WU_CONSTANT_WEIGHT, "DENDELAY": WU_DENDRITIC_DELAY,
            "STDP": WU_STDP}
CONN_KINDS = {"SPARSE": CONN_SPARSE, "BITMASK": CONN_BITMASK, "DENSE": CONN_DENSE,
              "PROCEDURAL": CONN_PROCEDURAL}
INIT_KINDS = {"Constant": INIT_CONSTANT, "Uniform": INIT_UNIFORM, "Normal": INIT_NORMAL,
              "NormalClipped": INIT_NORMAL_CLIPPED, "NormalClippedDelay": INIT_NORMAL_CLIPPED_DELAY}
CONNECT_KINDS = {"FixedProbability": CONNECT_FIXED_PROBABILITY,
                 "FixedProbabilityNoAutapse": CONNECT_FIXED_PROBABILITY_NO_AUTAPSE,
                 "FixedNumberTotalWithReplacement": CONNECT_FIXED_NUMBER_TOTAL,
                 "FixedNumberPreWithReplacement": CONNECT_FIXED_NUMBER_PRE,
                 "FixedNumberPostWithReplacement": CONNECT_FIXED_NUMBER_POST}


class Psm(C.Structure):
    _fields_ = [("model", C.c_uint32), ("max_den_delay", C.c_uint32), ("params", C.c_float * 4),
                ("out_post", C.c_void_p), ("den_delay", C.c_void_p)]


class CurrentSourceDesc(C.Structure):
    _fields_ = [("model", C.c_uint32), ("rng_stream", C.c_uint32), ("params", C.c_float * 4),
                ("var0", C.c_void_p)]


class NeuronGroupDesc(C.Structure):
    _fields_ = [("model", C.c_uint32), ("num_neurons", C.c_uint32), ("num_delay_slots", C.c_uint32),
                ("num_psm", C.c_uint32), ("num_cs", C.c_uint32), ("rng_stream", C.c_uint32),
                ("first_neuron", C.c_uint32), ("num_update", C.c_uint32),
                ("params", C.c_float * MAX_PARAMS), ("vars", C.c_void_p * MAX_VARS),
                ("egp", C.c_void_p), ("spk_cnt", C.c_void_p), ("spk", C.c_void_p),
                ("spike_times", C.c_void_p), ("record_spk", C.c_void_p),
                ("psm", Psm * MAX_PSM), ("cs", CurrentSourceDesc * MAX_CS),
                ("spk_slot_stride", C.c_uint32), ("reserved", C.c_uint32), ("spk_tag", C.c_void_p),
                ("spk_wire", C.c_void_p)]


class SynapseGroupDesc(C.Structure):
    _fields_ = [("connectivity", C.c_uint32), ("wu_model", C.c_uint32), ("num_src", C.c_uint32),
                ("num_trg", C.c_uint32), ("row_stride", C.c_uint32), ("ind_bytes", C.c_uint32),
                ("axonal_delay", C.c_uint32), ("back_prop_delay", C.c_uint32),
                ("src_delay_slots", C.c_uint32), ("trg_delay_slots", C.c_uint32),
                ("max_den_delay", C.c_uint32), ("col_stride", C.c_uint32),
                ("wu_params", C.c_float * MAX_PARAMS),
                ("row_length", C.c_void_p), ("ind", C.c_void_p), ("g", C.c_void_p), ("d", C.c_void_p),
                ("gp", C.c_void_p), ("col_length", C.c_void_p), ("remap", C.c_void_p),
                ("src_spk_cnt", C.c_void_p), ("src_spk", C.c_void_p),
                ("trg_spk_cnt", C.c_void_p), ("trg_spk", C.c_void_p),
                ("src_spike_times", C.c_void_p), ("trg_spike_times", C.c_void_p),
                ("out_post", C.c_void_p), ("den_delay", C.c_void_p),
                ("proc_connect", C.c_uint32), ("proc_weight_init", C.c_uint32),
                ("rng_stream", C.c_uint32), ("proc_weight_stream", C.c_uint32),
                ("proc_connect_params", C.c_float * 4), ("proc_weight_params", C.c_float * 4),
                ("src_sections", C.c_uint32), ("src_spk_slot_stride", C.c_uint32),
                ("src_cnt_section_stride", C.c_uint64), ("src_spk_section_stride", C.c_uint64),
                ("src_spk_tag", C.c_void_p), ("src_spk_wire", C.c_void_p)]


class CustomUpdateDesc(C.Structure):
    _fields_ = [("op", C.c_uint32), ("broadcast", C.c_uint32), ("num_elements", C.c_uint64),
                ("scale", C.c_float), ("reserved", C.c_uint32), ("source", C.c_void_p),
                ("target", C.c_void_p)]


LIB_NAME = "libgenn_b200.so"


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", LIB_NAME)


_PROTOTYPES = {
    "b200_runner_create": [C.c_int, C.c_double, C.c_uint64, C.c_uint32, C.POINTER(C.c_void_p)],
    "b200_runner_destroy": [C.c_void_p],
    "b200_device_count": [C.POINTER(C.c_int)],
    "b200_array_alloc": [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)],
    "b200_array_free": [C.c_void_p, C.c_void_p],
    "b200_host_alloc": [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)],
    "b200_host_free": [C.c_void_p, C.c_void_p],
    "b200_array_push": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t],
    "b200_array_pull": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t],
    "b200_array_memset": [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t],
    "b200_exchange_alloc": [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)],
    "b200_compact_words": [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p],
    "b200_timed_begin": [C.c_void_p],
    "b200_timed_end": [C.c_void_p, C.POINTER(C.c_float)],
    "b200_nccl_unique_id": [C.c_void_p],
    "b200_nccl_init": [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32],
    "b200_exchange_bytes": [C.c_void_p, C.POINTER(C.c_size_t)],
    "b200_exchange_get_handle": [C.c_void_p, C.c_void_p],
    "b200_exchange_open_peer": [C.c_void_p, C.c_uint32, C.c_void_p],
    "b200_exchange_set_peer": [C.c_void_p, C.c_uint32, C.c_void_p],
    "b200_exchange_configure": [C.c_void_p, C.c_uint32, C.c_uint32],
    "b200_push_neuron_update_group": [C.c_void_p, C.c_uint32, C.POINTER(NeuronGroupDesc)],
    "b200_push_synapse_group": [C.c_void_p, C.c_uint32, C.POINTER(SynapseGroupDesc)],
    "b200_validate_synapse_group": [C.POINTER(SynapseGroupDesc)],
    "b200_push_custom_update": [C.c_void_p, C.c_char_p, C.c_uint32, C.POINTER(CustomUpdateDesc)],
    "b200_initialize": [C.c_void_p],
    "b200_initialize_sparse": [C.c_void_p],
    "b200_init_var": [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32,
                      C.POINTER(C.c_float), C.c_uint32],
    "b200_init_sparse_connectivity": [C.c_void_p, C.c_uint32, C.POINTER(C.c_float), C.c_uint32, C.c_uint32,
                                      C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p,
                                      C.c_void_p, C.c_uint32],
    "b200_init_sparse_vars": [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32,
                              C.c_uint32, C.POINTER(C.c_float), C.c_uint32],
    "b200_build_remap": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                         C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p],
    "b200_update_synapses": [C.c_void_p],
    "b200_update_neurons": [C.c_void_p, C.c_uint64],
    "b200_step_time": [C.c_void_p, C.c_uint64, C.c_uint64],
    "b200_near_export": [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint64), C.c_uint32],
    "b200_near_import": [C.c_void_p, C.c_uint32, C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)],
    "b200_near_finish": [C.c_void_p, C.c_int],
    "b200_custom_update": [C.c_void_p, C.c_char_p],
    "b200_custom_update_reduce": [C.c_void_p, C.c_char_p],
    "b200_custom_update_broadcast": [C.c_void_p, C.c_char_p],
    "b200_synchronize": [C.c_void_p],
    "b200_get_timestep": [C.c_void_p, C.POINTER(C.c_uint64)],
    "b200_set_timestep": [C.c_void_p, C.c_uint64],
    "b200_get_steps_done": [C.c_void_p, C.POINTER(C.c_uint64)],
    "b200_enable_timing": [C.c_void_p, C.c_int],
    "b200_get_timer": [C.c_void_p, C.c_char_p, C.POINTER(C.c_double)],
    "b200_get_kernel_launches": [C.c_void_p, C.POINTER(C.c_uint64)],
    "b200_step_time_timed": [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(C.c_float)],
    "b200_get_counter": [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64)],
    "b200_set_option": [C.c_void_p, C.c_char_p, C.c_double],
    "b200_reset_timers": [C.c_void_p],
    "b200_get_cta_cycles": [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32)],
    "b200_get_step_path": [C.c_void_p, C.POINTER(C.c_int), C.c_char_p, C.c_size_t],
    "b200_update_neurons_noalloc": [C.c_int, C.c_void_p, C.POINTER(NeuronGroupDesc), C.c_uint32, C.c_uint32,
                                    C.c_double, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64],
    "b200_noalloc_check": [C.c_int, C.c_void_p],
}

_lib = None


class B200Error(RuntimeError):
    pass


def load_library():
    """Load the CUDA library.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise B200Error(f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                        "(there is no CPU fallback)")
    lib = C.CDLL(path)
    for name, argtypes in _PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int
    lib.b200_last_error.argtypes = []
    lib.b200_last_error.restype = C.c_char_p
    lib.b200_noalloc_last_error.argtypes = []
    lib.b200_noalloc_last_error.restype = C.c_char_p
    _lib = lib
    return lib


def check(status: int):
    if status != 0:
        msg = _lib.b200_last_error().decode() if _lib is not None else "?"
        raise B200Error(f"b200 error {status}: {msg}")


def exported_symbols():
    return list(_PROTOTYPES.keys()) + ["b200_last_error", "b200_noalloc_last_error"]
