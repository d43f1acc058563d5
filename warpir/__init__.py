"""Drop-in alias: ``warpir.*`` resolves to the B200 backend ``warpir_b200.*``.

Tile programs written for the reference import ``warpir.ir``,
``warpir.printing``, ``warpir.lowering`` and ``warpir.passes.modulo_scheduler``
(reference: tests/gemm_baseline_v2.py:13-29,93-95); this package makes those
names point at the sm_100a implementation so such programs run unchanged.
"""
import importlib as _importlib
import sys as _sys

_SUBMODULES = (
    "ir", "ir.types", "ir.ops",
    "printing", "printing.printer",
    "lowering", "lowering.lowering",
    "passes", "passes.modulo_scheduler", "passes.warp_assigner",
    "runtime",
)

for _name in _SUBMODULES:
    _mod = _importlib.import_module("warpir_b200." + _name)
    _sys.modules[__name__ + "." + _name] = _mod
    _parent, _, _leaf = _name.rpartition(".")
    _owner = _sys.modules[__name__ + ("." + _parent if _parent else "")]
    setattr(_owner, _leaf, _mod)
del _name, _mod, _parent, _leaf, _owner
