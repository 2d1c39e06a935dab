"""Registers the B200 backend with an installed PyGeNN.

PyGeNN discovers backends from a fixed list (pygenn/genn_model.py:106-120: cuda, hip,
single_threaded_cpu).  `register()` imports the `b200_backend` extension module (built from
genn_b200/backend/pygennBackend.cc against the same GeNN library PyGeNN was built with) and adds it
to that table under the name "b200", first in the order of preference, so that

    import genn_b200.pygenn_plugin as plugin; plugin.register()
    model = GeNNModel("float", "net", backend="b200")

builds, loads and steps the model on the B200 backend through PyGeNN's unmodified code path."""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys


def register(module_path: str | None = None, name: str = "b200"):
    """`module_path`: the built extension (b200_backend*.so); default: next to PyGeNN's own
    backend modules, else genn_b200/backend/."""
    import pygenn
    from pygenn import genn_model
    if name in genn_model.backend_modules:
        return genn_model.backend_modules[name]
    module = None
    if module_path is None:
        try:
            module = importlib.import_module("pygenn.b200_backend")
        except ImportError:
            here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "backend")
            found = [f for f in os.listdir(here) if f.startswith("b200_backend") and f.endswith(".so")]
            if not found:
                raise ImportError("b200_backend extension module has not been built")
            module_path = os.path.join(here, found[0])
    if module is None:
        spec = importlib.util.spec_from_file_location("pygenn.b200_backend", module_path)
        module = importlib.util.module_from_spec(spec)
        sys.modules["pygenn.b200_backend"] = module
        spec.loader.exec_module(module)
    genn_model.backend_modules[name] = module
    genn_model.backend_modules.move_to_end(name, last=False)
    return module
