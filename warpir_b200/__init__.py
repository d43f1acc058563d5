"""B200-native backend for WarpIR's hot path: bf16 GEMM and attention forward.

``warpir_b200.ir`` / ``.printing`` keep the reference's tile-IR builder and
printer API; ``.lowering`` and ``.passes`` target sm_100a (TMA, mbarrier rings,
``tcgen05.mma`` into tensor memory); ``.runtime`` binds the C-ABI launcher
(``libwarpir_b200.so``) through ``ctypes``.
"""
__version__ = "0.1.0"
