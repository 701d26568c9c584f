"""Shared driver of the split-KV decode-attention parity checks (imported by the pytest files and
run as a script in fresh processes by test_decode_attention_stress_gpu.py).

Before every launch the library's scratch buffers are overwritten with 0xFF bytes (NaN patterns)
and `out` is created full of NaN: a split that is skipped, a partial slot that is read without
having been written, or an output row that no CTA stores shows up as NaN instead of hiding behind
zeros or behind the identical numbers a previous call left in the same place."""
import ctypes
import math
import sys

import numpy as np


def ref_of(t):
    return ctypes.byref(t._handle.c())


def decode(q, kc, vc, ctx, splits=0, ctx_on_device=False, table=None, entry=None):
    from kandle_b200 import core, lib
    from kandle_b200.core import Tensor
    B, Hq, _, D = q.shape
    tq, tk, tv = Tensor(q, dtype="bfloat16"), Tensor(kc, dtype="bfloat16"), Tensor(vc, dtype="bfloat16")
    out = Tensor(np.full((B, Hq, 1, D), np.nan, np.float32), dtype="bfloat16")
    tctx = Tensor(np.array([ctx], np.int32)) if ctx_on_device else None
    scale = ctypes.c_float(1.0 / math.sqrt(D))
    lib.call("kd_debug_fill_scratch", 0xFF)
    if table is None:
        lib.call(entry or "kd_attention_decode", ref_of(tq), ref_of(tk), ref_of(tv), ref_of(tctx) if tctx else None,
                 0 if ctx_on_device else int(ctx), scale, splits, ref_of(out))
    else:
        tt = Tensor(table.astype(np.int32))
        lib.call("kd_attention_decode_paged", ref_of(tq), ref_of(tk), ref_of(tv), ref_of(tt), ref_of(tctx) if tctx else None,
                 0 if ctx_on_device else int(ctx), scale, splits, ref_of(out))
    return out.dataAsync()


def check(got, ref, rel=2e-2, what=""):
    err = np.abs(got - ref)
    bound = rel * np.abs(ref).max()
    if not (err.max() <= bound):          # NaN fails this comparison too
        bad = np.argwhere(~(err <= bound))
        rows = sorted({(int(i[0]), int(i[1])) for i in bad})      # (sequence, query head) pairs that are off
        raise AssertionError(f"{what}: {np.nanmax(err):.3e} > {bound:.3e}; {len(bad)} elements off "
                             f"({int(np.isnan(got).sum())} NaN) in {len(rows)} (sequence, head) rows, first {rows[:8]}")


def run_case(oracle, b, hq, hkv, max_s, ctx, d, splits, device_ctx_first=False):
    from kandle_b200 import lib, synth
    q = lib.round_to_bf16(synth.normal("q", (b, hq, 1, d)))
    kc = lib.round_to_bf16(synth.normal("kc", (b, hkv, max_s, d)))
    vc = lib.round_to_bf16(synth.normal("vc", (b, hkv, max_s, d)))
    ref = oracle.sdpa(q, kc[:, :, :ctx], vc[:, :, :ctx], is_causal=False)
    tag = f"[{b}-{hq}-{hkv}-{max_s}-{ctx}-{d}-{splits}]"
    for on_device in ((True, False) if device_ctx_first else (False, True)):
        check(decode(q, kc, vc, ctx, splits, ctx_on_device=on_device), ref, what=f"{tag} ctx_on_device={on_device}")


# Ragged shapes: the last key tile holds one key (ctx = 1 mod 64), one split, few splits, as many
# splits as the grid allows (0 = automatic), 1/2/4/8 query heads per KV head, both head sizes.
RAGGED = [
    (4, 16, 8, 2320, 2049, 128, 0), (4, 16, 8, 2320, 2049, 128, 9), (2, 16, 4, 1100, 1025, 128, 2),
    (3, 8, 8, 700, 641, 64, 1), (2, 32, 4, 900, 833, 128, 0), (1, 16, 8, 4200, 4097, 64, 9),
    (4, 8, 2, 320, 257, 128, 2), (2, 16, 8, 2320, 2176, 128, 0), (5, 4, 4, 200, 65, 64, 0),
]

if __name__ == "__main__":
    # python tests/decode_attention_cases.py <rotation>: the first launch of this process is the checked one
    import os
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import kandle_b200
    from oracle import oracle as orc
    orc.build()
    kandle_b200.init(0)
    rot = int(sys.argv[1]) if len(sys.argv) > 1 else 0
    cases = RAGGED[rot % len(RAGGED):] + RAGGED[:rot % len(RAGGED)]
    for i, c in enumerate(cases):
        run_case(orc, *c, device_ctx_first=bool((rot + i) & 1))
    print(f"decode attention: {len(cases)} ragged cases ok (rotation {rot})")
