"""The two tile programs of the hot path, written against ``warpir_b200.ir``.

With default arguments they build exactly the kernels of the reference's
``tests/gemm_baseline_v2.py:31-88`` (``build_gemm_kernel``) and
``tests/attention_baseline.py:46-186`` (``build_attention_kernel``): same value
names, types, op order and printed text.  The keyword arguments generalise what
the reference hard-codes (64-wide tiles, head dimension 64, row-major B) so the
same builders describe the tile shapes the sm_100a backend actually runs.
"""
from __future__ import annotations

import math

from .ir import (ColVecType, ForOp, GPUType, GlobalType, IntType, IterArg, Kernel,
                 RegTileType, SharedTileType, Value)
from . import ir as _ir

LOG2E = 1.44269504089  # the constant the reference folds into its scale (attention_baseline.py:43)


def _global_of(tile: SharedTileType) -> GlobalType:
    return GlobalType(data_type=GPUType.bf16, sub_tile_type=tile, batch=1, depth=1, rows=-1, cols=-1)


def build_gemm_kernel(block_m: int = 64, block_n: int = 64, block_k: int = 64,
                      b_k_major: bool = False) -> Kernel:
    """``C = A @ B`` as a k-loop of TMA loads and one MMA per step.

    ``b_k_major=False``: B is ``[K, N]`` row-major and tiles are fetched at
    ``(i, blockIdx.x)`` (the reference's program).  ``b_k_major=True``: B is
    stored ``[N, K]`` and the MMA takes ``transpose_b``.
    """
    a_tile = SharedTileType(GPUType.bf16, block_m, block_k)
    b_tile = (SharedTileType(GPUType.bf16, block_n, block_k) if b_k_major
              else SharedTileType(GPUType.bf16, block_k, block_n))
    c_tile = SharedTileType(GPUType.bf16, block_m, block_n)
    acc_t = RegTileType(GPUType.fp32, block_m // 4, block_n)  # rows per warp of a 4-warp group
    int_t = IntType()

    A, B = Value("A", _global_of(a_tile)), Value("B", _global_of(b_tile))
    C, N = Value("C_global", _global_of(c_tile)), Value("N", int_t)
    by, bx, i = Value("blockIdx.y", int_t), Value("blockIdx.x", int_t), Value("i", int_t)
    c_init, c_accum, c_final, c_new = (Value(n, acc_t) for n in ("c_init", "c_accum", "c_final", "c_new"))
    a_s, b_s = Value("a_shared", a_tile), Value("b_shared", b_tile)

    b_coords = (0, 0, bx, i) if b_k_major else (0, 0, i, bx)
    loop = ForOp(
        induction_var=i, start=0, stop=N, step=1, tile_size=block_k,
        iter_args=(IterArg(block_arg=c_accum, init=c_init),),
        body=(
            _ir.TMALoadOp(result=a_s, source=A, coords=(0, 0, by, i)),
            _ir.TMALoadOp(result=b_s, source=B, coords=b_coords),
            _ir.WaitOp(values=(a_s, b_s)),
            _ir.MMAOp(result=c_new, a=a_s, b=b_s, accum=c_accum, transpose_b=b_k_major),
            _ir.YieldOp(values=(c_new,)),
        ),
        results=(c_final,),
    )
    return Kernel(
        name="gemm", inputs=(A, B, N), outputs=(C,),
        body=(_ir.ZeroOp(result=c_init), loop,
              _ir.TMAStoreOp(source=c_final, dest=C, coords=(0, 0, by, bx))),
    )


def build_attention_kernel(head_dim: int = 64, block_q: int = 64, block_kv: int = 64,
                           scale: float | None = None) -> Kernel:
    """Single-head non-causal attention forward with an online base-2 softmax.

    ``scale`` is the factor applied to the raw scores *inside* ``exp2``; the
    default ``log2(e) / sqrt(head_dim)`` reproduces the reference's ``SCALE``
    (attention_baseline.py:42-43) for ``head_dim=64``.
    """
    if scale is None:
        scale = (1.0 / math.sqrt(head_dim)) * LOG2E
    q_tile = SharedTileType(GPUType.bf16, block_q, head_dim)
    kv_tile = SharedTileType(GPUType.bf16, block_kv, head_dim)
    s_t = RegTileType(GPUType.fp32, block_q // 4, block_kv)
    p_t = RegTileType(GPUType.bf16, block_q // 4, block_kv)
    o_t = RegTileType(GPUType.fp32, block_q // 4, head_dim)
    vec_t = ColVecType(GPUType.fp32, block_q // 4, block_kv)
    int_t = IntType()
    gq, gkv = _global_of(q_tile), _global_of(kv_tile)

    def vals(t, *names):
        return tuple(Value(n, t) for n in names)

    Q = Value("Q", gq)
    K, V = vals(gkv, "K", "V")
    O, N = Value("O", gq), Value("N", int_t)
    bx, i = vals(int_t, "blockIdx.x", "i")
    q_s = Value("q_shared", q_tile)
    k_s, v_s = vals(kv_tile, "k_shared", "v_shared")
    o_init, o_acc, o_resc, o_new, o_final, o_norm = vals(
        o_t, "o_init", "o_accum", "o_rescaled", "o_new", "o_final", "o_norm")
    (m_init, l_init, m_vec, l_vec, m_prev, m_new, m_new_sc, m_prev_sc, corr_diff, corr,
     l_resc, l_new, m_final, l_final) = vals(
        vec_t, "max_init", "norm_init", "max_vec", "norm_vec", "max_prev", "max_new",
        "max_new_sc", "max_prev_sc", "corr_diff", "correction", "norm_rescaled", "norm_new",
        "max_final", "norm_final")
    att_zero, att, att_sc, att_sh, p32 = vals(
        s_t, "att_zero", "att", "att_scaled", "att_shifted", "P_fp32")
    p16 = Value("P_bf16", p_t)

    body = (
        _ir.TMALoadOp(result=k_s, source=K, coords=(0, 0, i, 0)),
        _ir.TMALoadOp(result=v_s, source=V, coords=(0, 0, i, 0)),
        _ir.WaitOp(values=(k_s, v_s)),
        _ir.ZeroOp(result=att_zero),
        _ir.MMAOp(result=att, a=q_s, b=k_s, accum=att_zero, transpose_b=True),
        _ir.CopyOp(result=m_prev, input=m_vec),
        _ir.RowMaxOp(result=m_new, tile=att, prev=m_vec),
        _ir.MulScalarOp(result=att_sc, input=att, scalar=scale),
        _ir.MulScalarOp(result=m_new_sc, input=m_new, scalar=scale),
        _ir.MulScalarOp(result=m_prev_sc, input=m_prev, scalar=scale),
        _ir.SubRowOp(result=att_sh, tile=att_sc, vec=m_new_sc),
        _ir.Exp2Op(result=p32, input=att_sh),
        _ir.SubOp(result=corr_diff, a=m_prev_sc, b=m_new_sc),
        _ir.Exp2Op(result=corr, input=corr_diff),
        _ir.MulOp(result=l_resc, a=l_vec, b=corr),
        _ir.RowSumOp(result=l_new, tile=p32, prev=l_resc),
        _ir.MulRowOp(result=o_resc, tile=o_acc, vec=corr),
        _ir.CopyOp(result=p16, input=p32),
        _ir.MMAOp(result=o_new, a=p16, b=v_s, accum=o_resc),
        _ir.YieldOp(values=(o_new, m_new, l_new)),
    )
    loop = ForOp(
        induction_var=i, start=0, stop=N, step=1, tile_size=block_kv,
        iter_args=(IterArg(o_acc, o_init), IterArg(m_vec, m_init), IterArg(l_vec, l_init)),
        body=body, results=(o_final, m_final, l_final),
    )
    return Kernel(
        name="attention_fwd", inputs=(Q, K, V, N), outputs=(O,),
        body=(
            _ir.TMALoadOp(result=q_s, source=Q, coords=(0, 0, bx, 0)),
            _ir.WaitOp(values=(q_s,)),
            _ir.ZeroOp(result=o_init),
            _ir.NegInftyOp(result=m_init),
            _ir.ZeroOp(result=l_init),
            loop,
            _ir.DivRowOp(result=o_norm, tile=o_final, vec=l_final),
            _ir.TMAStoreOp(source=o_norm, dest=O, coords=(0, 0, bx, 0)),
        ),
    )
