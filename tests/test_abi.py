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
