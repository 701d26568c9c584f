"""GPU parity of the split-KV decode attention (contiguous and paged KV cache) against the CPU
oracle's single-row attention on the cache prefix.  bf16 bound as for the prefill kernel:
max-abs <= 2e-2 * max|ref|."""
import ctypes
import math

import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


def _ref(q):
    return ctypes.byref(q._handle.c())


def _decode(q, kc, vc, ctx, splits=0, ctx_on_device=False, table=None):
    B, Hq, _, D = q.shape
    tq, tk, tv = Tensor(q, dtype="bfloat16"), Tensor(kc, dtype="bfloat16"), Tensor(vc, dtype="bfloat16")
    out = core.empty((B, Hq, 1, D), "bfloat16")
    tctx = Tensor(np.array([ctx], np.int32)) if ctx_on_device else None
    scale = ctypes.c_float(1.0 / math.sqrt(D))
    if table is None:
        lib.call("kd_attention_decode", _ref(tq), _ref(tk), _ref(tv), _ref(tctx) if tctx else None, int(ctx), scale, splits, _ref(out))
    else:
        tt = Tensor(table.astype(np.int32))
        lib.call("kd_attention_decode_paged", _ref(tq), _ref(tk), _ref(tv), _ref(tt), _ref(tctx) if tctx else None, int(ctx),
                 scale, splits, _ref(out))
    return out.dataAsync()


def _check(got, ref, rel=2e-2):
    err = np.abs(got - ref).max()
    assert err <= rel * np.abs(ref).max(), f"{err:.3e} > {rel * np.abs(ref).max():.3e}"


@pytest.mark.parametrize("b,hq,hkv,max_s,ctx,d,splits", [
    (2, 16, 8, 512, 300, 128, 0), (3, 4, 4, 256, 256, 128, 1), (1, 8, 2, 1024, 1, 128, 4), (4, 16, 8, 2320, 2049, 128, 0),
    (2, 12, 12, 640, 129, 64, 3), (1, 32, 8, 384, 128, 128, 8), (2, 2, 1, 128, 77, 64, 0)])
def test_decode_attention_contiguous_cache(backend, oracle, b, hq, hkv, max_s, ctx, d, splits):
    q = lib.round_to_bf16(synth.normal("q", (b, hq, 1, d)))
    kc = lib.round_to_bf16(synth.normal("kc", (b, hkv, max_s, d)))
    vc = lib.round_to_bf16(synth.normal("vc", (b, hkv, max_s, d)))
    ref = oracle.sdpa(q, kc[:, :, :ctx], vc[:, :, :ctx], is_causal=False)
    _check(_decode(q, kc, vc, ctx, splits), ref)
    _check(_decode(q, kc, vc, ctx, splits, ctx_on_device=True), ref)


def test_decode_attention_equals_reference_expand_then_sdpa_path(backend, oracle):
    """The eager path (GQA expansion copy + flash_attention on prefix views) and the fused decode
    kernel agree."""
    b, hq, hkv, max_s, ctx, d = 2, 8, 4, 256, 200, 128
    q = lib.round_to_bf16(synth.normal("q", (b, hq, 1, d)))
    kc = lib.round_to_bf16(synth.normal("kc", (b, hkv, max_s, d)))
    vc = lib.round_to_bf16(synth.normal("vc", (b, hkv, max_s, d)))
    tk, tv = Tensor(kc, dtype="bfloat16"), Tensor(vc, dtype="bfloat16")
    pk, pv = tk.slice(f":, :, :{ctx}, :"), tv.slice(f":, :, :{ctx}, :")
    ek = pk.unsqueeze(2).expand((b, hkv, 2, ctx, d)).contiguous().view(b, hq, ctx, d)
    ev = pv.unsqueeze(2).expand((b, hkv, 2, ctx, d)).contiguous().view(b, hq, ctx, d)
    eager = core.scaledDotProductAttention(Tensor(q, dtype="bfloat16"), ek, ev, None, 0.0, False).dataAsync()
    fused = _decode(q, kc, vc, ctx)
    assert np.abs(eager - fused).max() <= 2e-2 * np.abs(eager).max()


def test_decode_attention_paged_cache(backend, oracle):
    b, hq, hkv, d, pages_per_seq, ctx = 3, 8, 4, 128, 5, 530
    n_pages = b * pages_per_seq + 2
    pool_k = lib.round_to_bf16(synth.normal("pk", (n_pages, hkv, 128, d)))
    pool_v = lib.round_to_bf16(synth.normal("pv", (n_pages, hkv, 128, d)))
    table = np.random.default_rng(5).permutation(n_pages)[: b * pages_per_seq].reshape(b, pages_per_seq)
    q = lib.round_to_bf16(synth.normal("q", (b, hq, 1, d)))
    kc = pool_k[table].transpose(0, 2, 1, 3, 4).reshape(b, hkv, pages_per_seq * 128, d)
    vc = pool_v[table].transpose(0, 2, 1, 3, 4).reshape(b, hkv, pages_per_seq * 128, d)
    ref = oracle.sdpa(q, kc[:, :, :ctx], vc[:, :, :ctx], is_causal=False)
    _check(_decode(q, pool_k, pool_v, ctx, 0, False, table), ref)
    _check(_decode(q, pool_k, pool_v, ctx, 2, True, table), ref)


def test_decode_attention_rejects_bad_arguments(backend):
    q = Tensor(synth.normal("q", (1, 4, 1, 128)), dtype="bfloat16")
    kc = Tensor(synth.normal("k", (1, 2, 64, 128)), dtype="bfloat16")
    out = core.empty((1, 4, 1, 128), "bfloat16")
    with pytest.raises(lib.KandleCudaError):      # context longer than the cache
        lib.call("kd_attention_decode", _ref(q), _ref(kc), _ref(kc), None, 65, ctypes.c_float(0.1), 0, _ref(out))
    with pytest.raises(lib.KandleCudaError):      # fp32 query
        q32 = Tensor(synth.normal("q", (1, 4, 1, 128)))
        lib.call("kd_attention_decode", _ref(q32), _ref(kc), _ref(kc), None, 8, ctypes.c_float(0.1), 0, _ref(out))


@pytest.mark.parametrize("b,hq,hkv,max_s,pos,d,splits,qkv_splits", [
    (32, 16, 8, 384, 300, 128, 0, 4),     # the benchmark's head layout, new token in the last (third) key tile
    (3, 16, 8, 512, 255, 128, 2, 2),      # new token is the last row of a tile; two KV splits, second one owns it
    (2, 4, 4, 256, 0, 128, 1, 1),         # first token of a sequence: the tile holds nothing but the new row
    (2, 12, 12, 640, 129, 64, 3, 3),      # head_dim 64, one query head per KV head
    (1, 32, 2, 384, 128, 128, 0, 1),      # 16 query heads per KV head: the whole 16-row Q tile is real
])
def test_decode_attention_with_fused_qkv_prologue(backend, b, hq, hkv, max_s, pos, d, splits, qkv_splits):
    """kd_attention_decode_qkv = kd_qkv_norm_rope_cachewrite + kd_attention_decode: the cache rows it
    writes must equal the two-kernel sequence bit for bit, its output up to the compiler's choice of
    fused multiply-adds in the two copies of the q-norm/RoPE arithmetic (a last-bit difference in one
    head's scale can flip the bf16 rounding of a query element: measured, one output row in 512)."""
    n_qkv = (hq + 2 * hkv) * d
    part = synth.normal("fq-part", (qkv_splits, b, n_qkv), 0.7)
    qw = lib.round_to_bf16(1.0 + synth.normal("fq-qw", (d,), 0.1))
    kw = lib.round_to_bf16(1.0 + synth.normal("fq-kw", (d,), 0.1))
    kc0 = lib.round_to_bf16(synth.normal("fq-kc", (b, hkv, max_s, d)))
    vc0 = lib.round_to_bf16(synth.normal("fq-vc", (b, hkv, max_s, d)))
    ang = synth.normal("fq-ang", (1, d // 2), 2.0)
    cos, sin = Tensor(np.cos(ang).astype(np.float32)), Tensor(np.sin(ang).astype(np.float32))
    tpart, tqw, tkw = Tensor(part), Tensor(qw, dtype="bfloat16"), Tensor(kw, dtype="bfloat16")
    tpos = Tensor(np.array([pos], np.int32))
    tctx = Tensor(np.array([pos + 1], np.int32))
    scale = ctypes.c_float(1.0 / math.sqrt(d))
    eps = ctypes.c_float(1e-6)
    # two kernels
    k1, v1 = Tensor(kc0, dtype="bfloat16"), Tensor(vc0, dtype="bfloat16")
    q1 = core.empty((b, 1, hq, d), "bfloat16")
    lib.call("kd_qkv_norm_rope_cachewrite", _ref(tpart), _ref(tqw), _ref(tkw), eps, _ref(cos), _ref(sin), _ref(k1), _ref(v1),
             _ref(tpos), 0, _ref(q1))
    o1 = core.empty((b, hq, 1, d), "bfloat16")
    q1v = q1.permute([0, 2, 1, 3])
    lib.call("kd_attention_decode", _ref(q1v), _ref(k1), _ref(v1), _ref(tctx), 0, scale, splits, _ref(o1))
    # one kernel
    k2, v2 = Tensor(kc0, dtype="bfloat16"), Tensor(vc0, dtype="bfloat16")
    o2 = core.empty((b, hq, 1, d), "bfloat16")
    lib.call("kd_attention_decode_qkv", _ref(tpart), _ref(tqw), _ref(tkw), eps, _ref(cos), _ref(sin), _ref(k2), _ref(v2),
             _ref(tpos), scale, splits, _ref(o2))
    backend.synchronize()
    assert np.array_equal(k2.dataAsync(), k1.dataAsync()) and np.array_equal(v2.dataAsync(), v1.dataAsync())
    assert not np.array_equal(k2.dataAsync()[:, :, pos], kc0[:, :, pos])        # the row was really written
    a, c = o2.dataAsync(), o1.dataAsync()
    rows_differ = (np.abs(a - c).max(-1) > 0).mean()
    assert np.abs(a - c).max() <= 2.0 ** -7 * np.abs(c).max() and rows_differ <= 0.01


def test_fused_qkv_prologue_reports_a_position_outside_the_cache(backend):
    b, hq, hkv, max_s, d = 1, 4, 2, 128, 128
    part = Tensor(synth.normal("fq-bad", (1, b, (hq + 2 * hkv) * d), 0.5))
    w = Tensor(np.ones(d, np.float32), dtype="bfloat16")
    cs = Tensor(np.ones((1, d // 2), np.float32))
    kc, vc = core.zeros((b, hkv, max_s, d), "bfloat16"), core.zeros((b, hkv, max_s, d), "bfloat16")
    out = core.empty((b, hq, 1, d), "bfloat16")
    bad = core.empty((b, hq, 1, d), "float32")
    with pytest.raises(lib.KandleCudaError):       # output must be bf16
        lib.call("kd_attention_decode_qkv", _ref(part), _ref(w), _ref(w), ctypes.c_float(1e-6), _ref(cs), _ref(cs), _ref(kc), _ref(vc),
                 _ref(Tensor(np.array([5], np.int32))), ctypes.c_float(0.1), 0, _ref(bad))
    with pytest.raises(lib.KandleCudaError):       # partial sums of the wrong width
        lib.call("kd_attention_decode_qkv", _ref(Tensor(np.zeros((1, b, 100), np.float32))), _ref(w), _ref(w), ctypes.c_float(1e-6),
                 _ref(cs), _ref(cs), _ref(kc), _ref(vc), _ref(Tensor(np.array([5], np.int32))), ctypes.c_float(0.1), 0, _ref(out))
