"""B200-native simulation backend for GeNN-style spiking neural network models.

The per-timestep hot path (neuron update, presynaptic update for SPARSE /
BITMASK / DENSE / PROCEDURAL connectivity, postsynaptic learning, the
initialisation kernels and batch-reduce custom updates) runs as hand-written
sm_100a CUDA kernels behind a C ABI (include/genn_b200.h); this package is the
host-side mirror of PyGeNN's model API on top of it.
"""
from .model import (GeNNModel, init_var, init_sparse_connectivity, init_postsynaptic,
                    init_weight_update)

__all__ = ["GeNNModel", "init_var", "init_sparse_connectivity", "init_postsynaptic",
           "init_weight_update"]
