"""Printer for tile programs.

Produces, character for character, the text of the reference's
``warpir/printing/printer.py:33-191`` (``format_kernel`` / ``print_kernel``):
every operand is written as ``%name: type``, ring buffers by bare name, slot
expressions as ``drain(+o, %m)`` / ``v % m`` / ``(v + o) % m``, and a loop as a
two-line header followed by a body indented by two levels.  The reference
switches on the op class; this printer is generic over the field roles that
each op class carries (``Op.roles``) and only special-cases the loop.  Ops it
does not know (no roles, not a loop) print nothing, as in the reference.
"""
from __future__ import annotations

from typing import List

from ..ir.ops import BufSlotExpr, ForOp, Kernel, Op


def _coord(c) -> str:
    return str(c) if isinstance(c, int) else repr(c)


def _slot(s) -> str:
    if isinstance(s, int):
        return str(s)
    assert isinstance(s, BufSlotExpr)
    if s.value is None:
        return f"drain(+{s.offset}, %{s.modulus})"
    if s.offset == 0:
        return f"{s.value!r} % {s.modulus}"
    return f"({s.value!r} + {s.offset}) % {s.modulus}"


def _operands(op: Op) -> List[str]:
    """Operand texts in field order, with a ``buf`` field fused to the ``slot``
    field that follows it (``name[slot]``)."""
    out: List[str] = []
    pending_buf = None
    for fname, role in op.roles:
        v = getattr(op, fname)
        if role == "result":
            continue
        if role == "use":
            out.append(repr(v))
        elif role == "uses":
            out.append(", ".join(repr(x) for x in v))
        elif role == "coords":
            out.append("[" + ", ".join(_coord(c) for c in v) + "]")
        elif role == "buf":
            pending_buf = v.name
        elif role == "bufs":
            out.append(", ".join(x.name for x in v))
        elif role == "slot":
            if pending_buf is not None:
                out.append(f"{pending_buf}[{_slot(v)}]")
                pending_buf = None
            else:
                out.append(f"slot={_slot(v)}")
        elif role == "attr":
            if isinstance(v, bool):
                if v:
                    out.append(f"{fname}=True")
            else:
                out.append(str(v))
    return out


def _emit(ops, depth: int, lines: List[str]) -> None:
    pad = "  " * depth
    for op in ops:
        if isinstance(op, ForOp):
            carried = ", ".join(f"{ia.block_arg!r} = {ia.init!r}" for ia in op.iter_args)
            results = ", ".join(repr(r) for r in op.results)
            tile = f" tile_size={op.tile_size}" if op.tile_size else ""
            lines.append(f"{pad}({results}) = for {op.induction_var!r} "
                         f"= {op.start} to {op.stop} step {op.step}{tile}")
            lines.append(f"{pad}    iter_args({carried}) {{")
            _emit(op.body, depth + 2, lines)
            lines.append(pad + "}")
            continue
        if not getattr(op, "roles", None):
            continue
        args = _operands(op)
        result = next((getattr(op, f) for f, r in op.roles if r == "result"), None)
        head = f"{result!r} = " if result is not None else ""
        if args:
            lines.append(f"{pad}{head}{op.mnemonic}({', '.join(args)})")
        elif result is not None:
            lines.append(f"{pad}{head}{op.mnemonic}")
        else:
            lines.append(f"{pad}{op.mnemonic}()")


def format_kernel(kernel: Kernel) -> str:
    """Readable SSA text of ``kernel``."""
    ins = ", ".join(repr(v) for v in kernel.inputs)
    outs = ", ".join(repr(v) for v in kernel.outputs)
    lines = [f"kernel {kernel.name}({ins}) -> ({outs}) {{"]
    _emit(kernel.body, 1, lines)
    lines.append("}")
    return "\n".join(lines)


def print_kernel(kernel: Kernel) -> None:
    """Write ``format_kernel(kernel)`` to stdout."""
    print(format_kernel(kernel))
