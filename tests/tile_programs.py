"""Tile programs beyond the two of the hot path, for the tests of the op-by-op emitter and
of the CPU interpreter.  Each builder returns ``(kernel, reference)`` where ``reference``
maps the input tensors (bf16, CPU) to the expected output in fp32, written directly in
torch from the mathematical definition (not through the interpreter)."""
from __future__ import annotations

import math

import torch

from warpir_b200 import ir as _ir
from warpir_b200.ir import (ColVecType, ForOp, GPUType, GlobalType, IntType, IterArg, Kernel,
                            RegTileType, SharedTileType, Value)

LOG2E = 1.4426950408889634


def _global(tile: SharedTileType) -> GlobalType:
    return GlobalType(data_type=GPUType.bf16, sub_tile_type=tile, batch=1, depth=1, rows=-1, cols=-1)


def _gemm_loop(bm, bn, bk, A, B, N, by, bx, acc_t, prefix="", bz=0):
    """c_final = sum_i A[bz, 0, by, i] @ B[bz, 0, i, bx] with B stored [K, N]."""
    a_tile, b_tile = SharedTileType(GPUType.bf16, bm, bk), SharedTileType(GPUType.bf16, bk, bn)
    i = Value(prefix + "i", IntType())
    a_s, b_s = Value(prefix + "a_shared", a_tile), Value(prefix + "b_shared", b_tile)
    c_init, c_acc, c_new, c_final = (Value(prefix + n, acc_t) for n in ("c_init", "c_accum", "c_new", "c_final"))
    loop = ForOp(induction_var=i, start=0, stop=N, step=1, tile_size=bk,
                 iter_args=(IterArg(c_acc, c_init),),
                 body=(_ir.TMALoadOp(a_s, A, (bz, 0, by, i)), _ir.TMALoadOp(b_s, B, (bz, 0, i, bx)),
                       _ir.WaitOp((a_s, b_s)), _ir.MMAOp(c_new, a_s, b_s, c_acc), _ir.YieldOp((c_new,))),
                 results=(c_final,))
    return [_ir.ZeroOp(c_init), loop], c_final


def scaled_gemm(bm=64, bn=64, bk=64, scale=0.5, batched=False):
    """C = scale * (A @ B): a GEMM whose result passes through an elementwise op, so the
    lowerer cannot hand it to the GEMM kernel.  ``batched``: one product per leading index
    (tensors [batch, 1, rows, cols], ``blockIdx.z`` picks the batch)."""
    acc_t = RegTileType(GPUType.fp32, bm // 4, bn)
    A = Value("A", _global(SharedTileType(GPUType.bf16, bm, bk)))
    B = Value("B", _global(SharedTileType(GPUType.bf16, bk, bn)))
    C = Value("C", _global(SharedTileType(GPUType.bf16, bm, bn)))
    N = Value("K_extent", IntType())
    by, bx = Value("blockIdx.y", IntType()), Value("blockIdx.x", IntType())
    bz = Value("blockIdx.z", IntType()) if batched else 0
    ops, c_final = _gemm_loop(bm, bn, bk, A, B, N, by, bx, acc_t, bz=bz)
    c_out = Value("c_scaled", acc_t)
    body = (*ops, _ir.MulScalarOp(c_out, c_final, scale), _ir.TMAStoreOp(c_out, C, (bz, 0, by, bx)))
    kernel = Kernel("scaled_gemm", inputs=(A, B, N), outputs=(C,), body=body)
    return kernel, lambda a, b: scale * (a.float() @ b.float())


def square_minus(bm=64, bn=64, bk=64):
    """C = T * T - T with T = A @ B: tile-by-tile ``mul`` and ``sub``."""
    acc_t = RegTileType(GPUType.fp32, bm // 4, bn)
    A = Value("A", _global(SharedTileType(GPUType.bf16, bm, bk)))
    B = Value("B", _global(SharedTileType(GPUType.bf16, bk, bn)))
    C = Value("C", _global(SharedTileType(GPUType.bf16, bm, bn)))
    N = Value("K_extent", IntType())
    by, bx = Value("blockIdx.y", IntType()), Value("blockIdx.x", IntType())
    ops, t = _gemm_loop(bm, bn, bk, A, B, N, by, bx, acc_t)
    sq, out = Value("t_squared", acc_t), Value("t_out", acc_t)
    body = (*ops, _ir.MulOp(sq, t, t), _ir.SubOp(out, sq, t), _ir.TMAStoreOp(out, C, (0, 0, by, bx)))
    kernel = Kernel("square_minus", inputs=(A, B, N), outputs=(C,), body=body)

    def ref(a, b):
        t = a.float() @ b.float()
        return t * t - t
    return kernel, ref


def row_softmax(block_q=64, block_kv=64, head_dim=128):
    """P = softmax(Q K^T / sqrt(d)) for one tile of keys: K-major B operand spanning two
    64-column chunks, ``neg_infty``, ``row_max``, ``sub_row``, ``exp2``, ``row_sum``, ``div_row``."""
    c = LOG2E / math.sqrt(head_dim)
    q_tile, k_tile = SharedTileType(GPUType.bf16, block_q, head_dim), SharedTileType(GPUType.bf16, block_kv, head_dim)
    p_tile = SharedTileType(GPUType.bf16, block_q, block_kv)
    s_t, vec_t = RegTileType(GPUType.fp32, block_q // 4, block_kv), ColVecType(GPUType.fp32, block_q // 4, block_kv)
    Q, K, P = Value("Q", _global(q_tile)), Value("K", _global(k_tile)), Value("P", _global(p_tile))
    bx = Value("blockIdx.x", IntType())
    q_s, k_s = Value("q_shared", q_tile), Value("k_shared", k_tile)
    zero, s, sc, sh, e, out = (Value(n, s_t) for n in ("s_zero", "s", "s_scaled", "s_shifted", "e", "p_out"))
    m0, m, l0, l = (Value(n, vec_t) for n in ("m_init", "m", "l_init", "l"))
    body = (
        _ir.TMALoadOp(q_s, Q, (0, 0, bx, 0)), _ir.TMALoadOp(k_s, K, (0, 0, 0, 0)), _ir.WaitOp((q_s, k_s)),
        _ir.ZeroOp(zero), _ir.MMAOp(s, q_s, k_s, zero, transpose_b=True),
        _ir.MulScalarOp(sc, s, c), _ir.NegInftyOp(m0), _ir.RowMaxOp(m, sc, m0), _ir.SubRowOp(sh, sc, m),
        _ir.Exp2Op(e, sh), _ir.ZeroOp(l0), _ir.RowSumOp(l, e, l0), _ir.DivRowOp(out, e, l),
        _ir.TMAStoreOp(out, P, (0, 0, bx, 0)),
    )
    kernel = Kernel("row_softmax", inputs=(Q, K), outputs=(P,), body=body)
    return kernel, lambda q, k: torch.softmax(q.float() @ k.float().t() / math.sqrt(head_dim), dim=-1)


def chained_gemm(bm=64, bk=64, mid=64, bn=128):
    """D = bf16(A @ B) @ W: the first product is rounded to bf16 in registers and fed to the
    second MMA as its A operand (register-tile A, as ``P V`` in attention), W stored [mid, bn]."""
    t_t, t16 = RegTileType(GPUType.fp32, bm // 4, mid), RegTileType(GPUType.bf16, bm // 4, mid)
    d_t = RegTileType(GPUType.fp32, bm // 4, bn)
    A = Value("A", _global(SharedTileType(GPUType.bf16, bm, bk)))
    B = Value("B", _global(SharedTileType(GPUType.bf16, bk, mid)))
    w_tile = SharedTileType(GPUType.bf16, mid, bn)
    W = Value("W", _global(w_tile))
    D = Value("D", _global(SharedTileType(GPUType.bf16, bm, bn)))
    N = Value("K_extent", IntType())
    by, bx = Value("blockIdx.y", IntType()), Value("blockIdx.x", IntType())
    ops, t = _gemm_loop(bm, mid, bk, A, B, N, by, 0, t_t)
    w_s = Value("w_shared", w_tile)
    tb, dz, d = Value("t_bf16", t16), Value("d_zero", d_t), Value("d", d_t)
    body = (*ops, _ir.TMALoadOp(w_s, W, (0, 0, 0, bx)), _ir.WaitOp((w_s,)), _ir.CopyOp(tb, t), _ir.ZeroOp(dz),
            _ir.MMAOp(d, tb, w_s, dz), _ir.TMAStoreOp(d, D, (0, 0, by, bx)))
    kernel = Kernel("chained_gemm", inputs=(A, B, W, N), outputs=(D,), body=body)

    def ref(a, b, w):
        t = (a.float() @ b.float()).to(torch.bfloat16).float()
        return t @ w.float()
    return kernel, ref


def op_by_op_cases():
    """Every program the GPU tests run through the op-by-op emitter, as
    ``id -> (kernel, force)``; ``force`` asks the lowerer to emit one of the two recognised
    programs op by op as well.  The build step compiles the same list ahead of time."""
    from warpir_b200.passes.modulo_scheduler import REFERENCE_MODEL, kernel_pass
    from warpir_b200.programs import build_attention_kernel, build_gemm_kernel
    return {
        "scaled_gemm_64": (scaled_gemm()[0], False),
        "scaled_gemm_128x128": (scaled_gemm(128, 128, 64)[0], False),
        "scaled_gemm_128x256": (scaled_gemm(128, 256, 64)[0], False),
        "scaled_gemm_batched": (scaled_gemm(batched=True)[0], False),
        "square_minus": (square_minus()[0], False),
        "row_softmax_d128": (row_softmax(64, 64, 128)[0], False),
        "row_softmax_q128_kv128": (row_softmax(128, 128, 64)[0], False),
        "chained_gemm": (chained_gemm()[0], False),
        "reference_gemm": (build_gemm_kernel(), True),
        "reference_gemm_pipelined": (kernel_pass(build_gemm_kernel(), REFERENCE_MODEL), True),
        "k_major_gemm_pipelined": (kernel_pass(build_gemm_kernel(block_n=64, b_k_major=True), REFERENCE_MODEL), True),
        "reference_attention": (build_attention_kernel(), True),
        "attention_d128": (build_attention_kernel(head_dim=128), True),
    }
