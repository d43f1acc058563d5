"""Regenerates the fixtures in this folder FROM THE REFERENCE ITSELF.

Run in a container that has the reference checkout (read-only) beside the repo:

    python tests/golden/make_golden.py <path to the reference checkout>

It imports the reference's own Python (its printer, its two tile programs, its
``_ref_attention``) and writes:

* ``printer_gemm.txt`` / ``printer_attention.txt`` -- ``format_kernel`` of the
  reference's GEMM and attention tile programs (reference:
  warpir/printing/printer.py:38-46, tests/gemm_baseline_v2.py:31,
  tests/attention_baseline.py:46);
* ``printer_gemm_pipelined.txt`` -- ``format_kernel`` of the reference's
  ``kernel_pass`` output (warpir/passes/modulo_scheduler.py:168).  That pass
  needs OR-tools CP-SAT, which is not installed; a stand-in ``cp_model`` is
  injected that solves the same model exactly for this instance (see
  ``_FakeCpModel``);
* ``gemm_small.npz`` -- seeded bf16 A, B and ``torch.mm(A.float(), B.float())``
  (the expression at tests/test_gemm_baseline.py:85);
* ``attention_small.npz`` -- seeded bf16 Q, K, V and the output of the reference's
  ``_ref_attention`` (tests/test_modal_attention.py:92-98), imported with the
  absent ``modal`` package stubbed out (it is only used for remote launch).

bf16 tensors are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import itertools
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


# ---------------------------------------------------------------------------
# stand-ins for packages the reference imports but that are absent here
# ---------------------------------------------------------------------------

def _stub_modal() -> None:
    m = types.ModuleType("modal")

    class _Chain:
        def __getattr__(self, _):
            return lambda *a, **k: self

    class _App:
        def __init__(self, *a, **k):
            pass

        def function(self, *a, **k):
            return lambda f: f

        def local_entrypoint(self, *a, **k):
            return lambda f: f

    m.Image = _Chain()
    m.App = _App
    sys.modules["modal"] = m


class _FakeCpModel:
    """Just enough of ``ortools.sat.python.cp_model`` for the reference's
    modulo scheduler.  The model it builds (modulo_scheduler.py:51-101) has one
    start variable per (unrolled copy, instruction), precedence constraints
    ``start >= end``, the recurrences ``start[k+1] == start[k] + ii``, one
    cumulative constraint per resource and minimises the makespan.  With ``ii``
    and the copy-0 starts chosen, everything else is determined, so the exact
    optimum is found by enumerating ``ii`` upward and the copy-0 starts, keeping
    the lexicographically first assignment of least makespan."""

    OPTIMAL, FEASIBLE, INFEASIBLE = 4, 2, 3

    class _Expr:
        def __init__(self, var=None, const=0, extra=None):
            self.var, self.const, self.extra = var, const, extra

        def __add__(self, o):
            if isinstance(o, _FakeCpModel._Expr):
                return _FakeCpModel._Expr(self.var, self.const + o.const, o.var)
            return _FakeCpModel._Expr(self.var, self.const + o, self.extra)

        def __ge__(self, o):
            return ("ge", self, o)

        def __eq__(self, o):  # noqa: PLR0124 - builds a constraint, like CP-SAT does
            return ("eq", self, o)

        __hash__ = object.__hash__

    class _Var(_Expr):
        def __init__(self, lo, hi, name):
            super().__init__(self, 0)
            self.lo, self.hi, self.name = lo, hi, name

    class _Interval:
        def __init__(self, start, size, name):
            self.start, self.size, self.name = start, size, name

        def start_expr(self):
            return self.start

        def end_expr(self):
            return self.start + self.size

    class CpModel:
        def __init__(self):
            self.vars, self.cons, self.cums, self.intervals = [], [], [], []
            self.makespan = None

        def new_int_var(self, lo, hi, name):
            v = _FakeCpModel._Var(lo, hi, name)
            self.vars.append(v)
            return v

        def new_interval_var(self, start, size, end, name):
            iv = _FakeCpModel._Interval(start, size, name)
            self.intervals.append(iv)
            return iv

        def add(self, c):
            self.cons.append(c)

        def add_cumulative(self, ivs, demands, cap):
            self.cums.append((list(ivs), cap))

        def add_max_equality(self, target, exprs):
            self.makespan = (target, list(exprs))

        def minimize(self, _):
            pass

    class _Params:
        log_search_progress = False

    class CpSolver:
        def __init__(self):
            self.parameters = _FakeCpModel._Params()
            self.assign = {}

        def value(self, e):
            if isinstance(e, _FakeCpModel._Expr):
                v = self.assign[e.var] + e.const
                if e.extra is not None:
                    v += self.assign[e.extra]
                return v
            return e

        def solve(self, model):
            F = _FakeCpModel
            ii = next(v for v in model.vars if v.name == "ii")
            starts = [iv.start for iv in model.intervals]
            depth0 = [s for s in starts if s.name.endswith("_0")]
            per_name = {}
            for s in starts:
                base, _, k = s.name.rpartition("_")
                per_name.setdefault(base, {})[int(k)] = s
            size_of = {iv.start: iv.size for iv in model.intervals}
            best = None
            horizon = max(v.hi for v in starts) + 1
            for iiv in range(ii.lo, ii.hi + 1):
                if best is not None and iiv * (len(next(iter(per_name.values()))) - 1) >= best[0]:
                    break
                ranges = [range(s.lo, min(s.hi, horizon) + 1) for s in depth0]
                for combo in itertools.product(*ranges):
                    a = {ii: iiv}
                    ok = True
                    for s0, v0 in zip(depth0, combo):
                        base = s0.name.rpartition("_")[0]
                        for k, s in per_name[base].items():
                            val = v0 + k * iiv
                            if val > s.hi:
                                ok = False
                                break
                            a[s] = val
                        if not ok:
                            break
                    if not ok:
                        continue
                    span = max(a[s] + size_of[s] for s in starts)
                    if best is not None and span >= best[0]:
                        continue
                    self.assign = a
                    if not all(self._holds(c) for c in model.cons):
                        continue
                    if not all(self._cum_ok(ivs, cap) for ivs, cap in model.cums):
                        continue
                    best = (span, dict(a))
                    horizon = span  # nothing starting later can win
            if best is None:
                return F.INFEASIBLE
            self.assign = best[1]
            self.assign[model.makespan[0]] = best[0]
            return F.OPTIMAL

        def _holds(self, c):
            kind, lhs, rhs = c
            l, r = self.value(lhs), self.value(rhs)
            return l >= r if kind == "ge" else l == r

        def _cum_ok(self, ivs, cap):
            events = []
            for iv in ivs:
                s = self.value(iv.start)
                events.append((s, 1))
                events.append((s + iv.size, -1))
            load = 0
            for _, d in sorted(events, key=lambda e: (e[0], e[1])):
                load += d
                if load > cap:
                    return False
            return True


def _stub_ortools() -> None:
    root = types.ModuleType("ortools")
    sat = types.ModuleType("ortools.sat")
    py = types.ModuleType("ortools.sat.python")
    cp = types.ModuleType("ortools.sat.python.cp_model")
    for name in ("CpModel", "CpSolver", "OPTIMAL", "FEASIBLE", "INFEASIBLE"):
        setattr(cp, name, getattr(_FakeCpModel, name))
    cp.IntervalVar = _FakeCpModel._Interval
    py.cp_model = cp
    sat.python = py
    root.sat = sat
    sys.modules.update({"ortools": root, "ortools.sat": sat,
                        "ortools.sat.python": py, "ortools.sat.python.cp_model": cp})


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    # the repo's own ``warpir`` alias must not shadow the reference's package
    for k in [k for k in sys.modules if k == "warpir" or k.startswith("warpir.")]:
        del sys.modules[k]
    _stub_modal()
    _stub_ortools()

    from tests.attention_baseline import build_attention_kernel
    from tests.gemm_baseline_v2 import build_gemm_kernel
    from warpir.printing import format_kernel
    import warpir
    assert Path(warpir.__file__).resolve().is_relative_to(Path(ref_root).resolve()), warpir.__file__

    (HERE / "printer_gemm.txt").write_text(format_kernel(build_gemm_kernel()) + "\n")
    (HERE / "printer_attention.txt").write_text(format_kernel(build_attention_kernel()) + "\n")

    from warpir.passes.modulo_scheduler import kernel_pass
    (HERE / "printer_gemm_pipelined.txt").write_text(
        format_kernel(kernel_pass(build_gemm_kernel())) + "\n")

    # GEMM: the expression at tests/test_gemm_baseline.py:85, on CPU tensors
    g = torch.Generator().manual_seed(0)
    A = torch.randn(128, 192, generator=g).to(torch.bfloat16)
    B = torch.randn(192, 64, generator=g).to(torch.bfloat16)
    ref = torch.mm(A.float(), B.float())
    np.savez_compressed(HERE / "gemm_small.npz", A=bits(A), B=bits(B), ref=ref.numpy())

    # attention: the reference's own _ref_attention (single head, non-causal, 1/sqrt(D))
    from tests.test_modal_attention import _ref_attention
    out = {}
    for tag, (N, D) in {"n256_d64": (256, 64), "n128_d128": (128, 128)}.items():
        g = torch.Generator().manual_seed(1)
        Q = torch.randn(N, D, generator=g).to(torch.bfloat16)
        K = torch.randn(N, D, generator=g).to(torch.bfloat16)
        V = torch.randn(N, D, generator=g).to(torch.bfloat16)
        O = _ref_attention(Q, K, V)
        out.update({f"{tag}_Q": bits(Q), f"{tag}_K": bits(K), f"{tag}_V": bits(V),
                    f"{tag}_O": bits(O)})
    np.savez_compressed(HERE / "attention_small.npz", **out)
    print("wrote", sorted(p.name for p in HERE.iterdir()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
