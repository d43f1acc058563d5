"""Event timeline of one CTA of the attention forward, from a debug build of the library.

    python -m warpir_b200.build --variant trace WIR_TRACE
    python -m warpir_b200.trace [--variant 1|4] [--causal] [--head-dim 64|128] [--from N --to M]

The kernels compiled with ``-DWIR_TRACE`` make a few threads of CTA (0, 0, 0) append
(event, index, clock64) records to a device buffer (``csrc/ptx.cuh``: ``WIR_TRACE_EVENT``).  This tool
launches the forward on one CTA per SM, reads the buffer back and prints the records in time order:
region 0 / 3 = the MMA-issuing warp(s), 1 / 2 = the softmax warpgroups of Q tile 0 / 1.  Events of the
softmax warps: 100 waits for the scores, 101 has them, 102 has loaded them from tensor memory,
103 has stored P and signalled it.  Events of the issuer (plus 10 for Q tile 1): 1 waits for P,
2 has it, 3 has issued P V, 4 has issued the next Q K^T.  A measurement aid; the product library has
no tracing in it."""
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
    args = ap.parse_args()
    import torch
    path = build.LIB_DIR / "libwarpir_b200_trace.so"
    if not path.exists():
        path = build.build_variant("trace", ["WIR_TRACE"])
    lib = ctypes.CDLL(str(path))
    vp, i64, ci, cf = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    lib.warpir_attn_fwd_bf16_ex.restype = ci
    lib.warpir_attn_fwd_bf16_ex.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, cf, ci, ci, ci, vp]
    lib.warpir_debug_set_trace.argtypes = [vp]
    regions, per = 8, 4096
    B, H, S, D = 1, 148, 2048, args.head_dim      # grid (8, 148, 1): a few waves; CTA (0, 0, 0) is traced
    Q = torch.randn(B, H, S, D, device="cuda").bfloat16()
    K, V, O = torch.randn_like(Q), torch.randn_like(Q), torch.empty_like(Q)
    buf = torch.zeros(2 * regions * per, dtype=torch.int64, device="cuda")

    def run():
        return lib.warpir_attn_fwd_bf16_ex(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), None, B, H, H, S, D,
                                           D ** -0.5, int(args.causal), args.variant, 0, None)
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
            events.append((clock, r, tag >> 32, tag & 0xffffffff))
    events.sort()
    t0 = events[0][0] if events else 0
    for clock, r, ev, idx in events:
        if args.lo <= idx < args.hi:
            print(f"{clock - t0:8d} region={r} event={ev:3d} block={idx}")


if __name__ == "__main__":
    main()
