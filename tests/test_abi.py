"""The C-ABI library loads and exports every symbol include/genn_b200.h declares
(no compute calls: this runs without a GPU)."""
import ctypes
import os
import re

import pytest

from genn_b200 import abi

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(REPO, "include", "genn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def library():
    if not os.path.exists(abi.library_path()):
        import __graft_entry__
        __graft_entry__.build()
    return ctypes.CDLL(abi.library_path())


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "b200_step_time" in names and "b200_push_synapse_group" in names
    assert len(names) >= 30


def test_library_exports_every_declared_symbol(library):
    missing = [n for n in declared_symbols() if not hasattr(library, n)]
    assert not missing, f"declared in genn_b200.h but not exported: {missing}"


def test_python_prototypes_cover_the_header(library):
    assert sorted(abi.exported_symbols()) == declared_symbols()


def test_descriptor_sizes_match_the_header():
    """ctypes mirrors must have the C layout (checked against sizes the C
    compiler reports for the same header)."""
    import subprocess
    import tempfile
    src = r'''
    #include <stdio.h>
    #include "genn_b200.h"
    int main(void) {
        printf("%zu %zu %zu %zu %zu\n", sizeof(b200_psm), sizeof(b200_current_source),
               sizeof(b200_neuron_group), sizeof(b200_synapse_group), sizeof(b200_custom_update_group));
        return 0;
    }'''
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.check_call(["/usr/bin/gcc", "-I", os.path.join(REPO, "include"), c, "-o", exe])
        sizes = [int(x) for x in subprocess.check_output([exe]).split()]
    assert sizes == [ctypes.sizeof(abi.Psm), ctypes.sizeof(abi.CurrentSourceDesc), ctypes.sizeof(abi.NeuronGroupDesc),
                     ctypes.sizeof(abi.SynapseGroupDesc), ctypes.sizeof(abi.CustomUpdateDesc)]


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(abi, "_lib", None)
    monkeypatch.setattr(abi, "library_path", lambda: "/nonexistent/libgenn_b200.so")
    with pytest.raises(abi.B200Error):
        abi.load_library()


# ---------------------------------------------------------------------------
# Descriptors the kernels could not take are refused when they are pushed
# (checked here without a GPU; none of them is ever handed to a kernel)
# ---------------------------------------------------------------------------
def _good_sparse():
    d = abi.SynapseGroupDesc()
    d.connectivity, d.wu_model = abi.CONN_SPARSE, abi.WU_STATIC_PULSE
    d.num_src, d.num_trg, d.row_stride, d.ind_bytes = 10, 20, 8, 4
    d.src_delay_slots, d.trg_delay_slots = 4, 4
    # any non-null, suitably aligned addresses: validation never dereferences them
    d.row_length, d.ind, d.g, d.out_post = 0x1000, 0x2000, 0x3000, 0x4000
    d.src_spk_cnt, d.src_spk = 0x5000, 0x6000
    return d


def _validate(library, d):
    library.b200_validate_synapse_group.argtypes = [ctypes.POINTER(abi.SynapseGroupDesc)]
    library.b200_validate_synapse_group.restype = ctypes.c_int
    return library.b200_validate_synapse_group(ctypes.byref(d))


def test_a_well_formed_descriptor_passes(library):
    assert _validate(library, _good_sparse()) == abi.OK


def _ring_without_delays(d):
    d.max_den_delay, d.den_delay = 16, 0x7000          # d missing


def _ring_on_static_pulse(d):
    d.max_den_delay, d.den_delay, d.d = 16, 0x7000, 0x8000


def _dendritic_delay_on_dense(d):
    d.connectivity, d.wu_model = abi.CONN_DENSE, abi.WU_DENDRITIC_DELAY
    d.max_den_delay, d.den_delay, d.d, d.out_post = 16, 0x7000, 0x8000, 0


def _ring_on_bitmask(d):
    d.connectivity, d.wu_model, d.gp, d.row_stride = abi.CONN_BITMASK, abi.WU_CONSTANT_WEIGHT, 0x9000, 32
    d.max_den_delay, d.den_delay, d.d = 16, 0x7000, 0x8000


def _no_out_post(d):
    d.out_post = 0


def _misaligned_g(d):
    d.g = 0x3004


def _misaligned_ind(d):
    d.ind = 0x2004


def _misaligned_narrow_ind(d):
    d.ind_bytes, d.ind = 2, 0x2002


def _misaligned_d(d):
    d.wu_model, d.max_den_delay, d.den_delay, d.d = abi.WU_DENDRITIC_DELAY, 16, 0x7000, 0x8001


def _back_prop_delay_too_long(d):
    d.wu_model = abi.WU_STDP
    d.src_spike_times, d.trg_spike_times, d.trg_spk, d.trg_spk_cnt = 0xA000, 0xB000, 0xC000, 0xD000
    d.col_length, d.remap = 0xE000, 0xF000
    d.back_prop_delay = 3                               # needs 5 slots, the queue has 4


def _axonal_delay_too_long(d):
    d.axonal_delay = 3


@pytest.mark.parametrize("spoil", [_ring_without_delays, _ring_on_static_pulse, _dendritic_delay_on_dense,
                                   _ring_on_bitmask, _no_out_post, _misaligned_g, _misaligned_ind,
                                   _misaligned_narrow_ind, _misaligned_d, _back_prop_delay_too_long,
                                   _axonal_delay_too_long], ids=lambda f: f.__name__.strip("_"))
def test_bad_descriptors_are_refused(library, spoil):
    d = _good_sparse()
    spoil(d)
    assert _validate(library, d) == abi.ERR_INVALID
    library.b200_last_error.restype = ctypes.c_char_p
    assert library.b200_last_error()
