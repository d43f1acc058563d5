"""Event timeline of one CTA of the attention forward or backward, from a debug build of the library.

    python -m warpir_b200.build --variant trace WIR_TRACE
    python -m warpir_b200.trace [--variant 1|4] [--causal] [--head-dim 64|128] [--from N --to M]
    python -m warpir_b200.trace --backward [--dq-only] [--library libwarpir_b200_trace.so] [--from N --to M]

The kernels compiled with ``-DWIR_TRACE`` make a few threads of CTA (0, 0, 0) append
(event, index, clock64) records to a device buffer (``csrc/ptx.cuh``: ``WIR_TRACE_EVENT``).  This tool
launches the forward on one CTA per SM, reads the buffer back and prints the records in time order:
region 0 / 3 = the MMA-issuing warp(s), 1 / 2 = the softmax warpgroups of Q tile 0 / 1.  Events of the
softmax warps: 100 waits for the scores, 101 has them, 102 has loaded them from tensor memory,
103 has stored P and signalled it.  Events of the issuer (plus 10 for Q tile 1): 1 waits for P,
2 has it, 3 has issued P V, 4 has issued the next Q K^T.

``--backward``: the two launches of the backward write the same regions, the second over the first, so
the timeline shown is that of the dK/dV launch unless ``--dq-only`` stops after the dQ launch.  The 128-row
kernel (the library's choice): region 0 = the MMA-issuing warp (0 a step begins, 1 has seen "P ready" (dQ launch:
T0 read), 2 has issued B1 (and the next scores if they had to wait for their tile), 3 has seen "dS ready", 4 has
issued B2 / B and the next dP), 1 / 2 = one thread of compute warpgroup 0 / 1 (10 a step begins, 11 T0 has
arrived, 15 T0 is loaded and released, 16 exponentials done, 13 T1 has arrived, 17 T1 is loaded, 12 P stored and
signalled (dK/dV launch), 14 dS stored and signalled; 90 set-up done, 91 prologue done, 92 accumulators complete),
3 = event 93, epilogue done.  With ``WARPIR_ATTN_BWD_ROWS=64`` the 64-row kernel runs instead (region 0: 0 waits
for P / dS of a step, 1 has them, 2 has issued stage 2, 3 has issued stage 1 of the step after next; compute:
10 waits for the scores, 11 has them, 12 has loaded a pass of 32 columns, 13 has stored P / dS, 14 has signalled).
``--library`` names another
debug build (e.g. one that also has ``WIR_BWD_ABLATE`` set).  A measurement aid; the product library
has no tracing in it."""
from __future__ import annotations

import argparse
import ctypes

from . import build


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--variant", type=int, default=4)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--from", dest="lo", type=int, default=0)
    ap.add_argument("--to", dest="hi", type=int, default=1 << 30)
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--dq-only", action="store_true")
    ap.add_argument("--library", default="libwarpir_b200_trace.so")
    args = ap.parse_args()
    import os
    if args.dq_only:
        os.environ["WARPIR_BWD_DQ_ONLY"] = "1"       # read by debug and measurement builds at every launch
    import torch
    path = build.LIB_DIR / args.library
    if not path.exists():
        path = build.build_variant("trace", ["WIR_TRACE"])
    lib = ctypes.CDLL(str(path))
    vp, i64, ci, cf = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    lib.warpir_attn_fwd_bf16_ex.restype = ci
    lib.warpir_attn_fwd_bf16_ex.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, cf, ci, ci, ci, vp]
    lib.warpir_attn_bwd_bf16.restype = ci
    lib.warpir_attn_bwd_bf16.argtypes = [vp] * 10 + [i64] * 5 + [cf, ci, ci, vp]
    lib.warpir_debug_set_trace.argtypes = [vp]
    regions, per = 8, 4096
    B, H, S, D = 1, 148, 2048, args.head_dim      # grid (8, 148, 1): a few waves; CTA (0, 0, 0) is traced
    Q = torch.randn(B, H, S, D, device="cuda").bfloat16()
    K, V, O = torch.randn_like(Q), torch.randn_like(Q), torch.empty_like(Q)
    buf = torch.zeros(2 * regions * per, dtype=torch.int64, device="cuda")

    def forward(lse=None):
        return lib.warpir_attn_fwd_bf16_ex(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), lse, B, H, H, S, D,
                                           D ** -0.5, int(args.causal), 0 if args.backward else args.variant, 0, None)
    run = forward
    if args.backward:
        L = torch.empty(B, H, S, device="cuda")
        dO = torch.randn_like(Q)
        dQ = torch.empty(B, H, S, D, device="cuda")
        dK, dV, delta = torch.empty_like(dQ), torch.empty_like(dQ), torch.empty(B * H * S, device="cuda")
        lib.warpir_debug_set_trace(None)
        if forward(L.data_ptr()) != 0:
            raise SystemExit("forward failed")

        def run():
            return lib.warpir_attn_bwd_bf16(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), dO.data_ptr(),
                                            L.data_ptr(), dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(), delta.data_ptr(),
                                            B, H, H, S, D, D ** -0.5, int(args.causal), 0, None)
    lib.warpir_debug_set_trace(None)
    run()
    run()
    torch.cuda.synchronize()
    lib.warpir_debug_set_trace(buf.data_ptr())
    rc = run()
    torch.cuda.synchronize()
    if rc != 0:
        raise SystemExit(f"launch failed: {rc}")
    host = buf.cpu().tolist()
    events = []
    for r in range(regions):
        for i in range(per):
            tag, clock = host[2 * (r * per + i)], host[2 * (r * per + i) + 1]
            if clock == 0:
                break
            if i > 0 and clock < host[2 * (r * per + i - 1) + 1]:
                break                              # left over from an earlier, longer launch
            events.append((clock, r, tag >> 32, tag & 0xffffffff))
    events.sort()
    t0 = events[0][0] if events else 0
    for clock, r, ev, idx in events:
        if args.lo <= idx < args.hi or 90 <= ev < 100:
            print(f"{clock - t0:8d} region={r} event={ev:3d} block={idx}")
    if args.backward:
        got = [c for c, r, ev, _ in events if r == 0 and ev == 1]
        if len(got) > 4:
            d = sorted(b - a for a, b in zip(got, got[1:]))
            print(f"issuing warp, clocks per step: median {d[len(d) // 2]} min {d[0]} max {d[-1]} over {len(d)} steps")


if __name__ == "__main__":
    main()
