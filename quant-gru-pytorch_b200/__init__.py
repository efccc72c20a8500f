"""B200-native integer quantized GRU forward: Python host side.

The directory name contains a hyphen, so the package is loaded under the module name
``quant_gru_pytorch_b200`` by ``__graft_entry__.load_package()`` (importlib), not by a plain
``import``.  Sub-modules:

``_cabi``      ctypes view of the C ABI declared in include/qgru.h and the library loader
``build``      nvcc build of csrc/ into libqgru_b200.so (sm_100a)
``params``     host data model: operator configs, quant params, ranges, JSON round trips
``gru_ops``    functions with the names and argument meaning of the reference's ``gru_ops``
               pybind module (pytorch/lib/gru_interface_binding.cc) for the integer path
``quant_gru``  ``QuantGRU``: the nn.GRU-compatible module of pytorch/quant_gru.py, hot path only
``sharding``   batch / direction partition over several GPUs (one process per GPU)
"""
from . import _cabi  # noqa: F401

__all__ = ["_cabi"]
