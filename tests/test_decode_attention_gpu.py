"""GPU parity of the split-KV decode attention (contiguous and paged KV cache) against the CPU
oracle's single-row attention on the cache prefix.  bf16 bound as for the prefill kernel:
max-abs <= 2e-2 * max|ref|."""
import ctypes
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


from decode_attention_cases import check as _check, decode as _decode, ref_of as _ref, run_case


@pytest.mark.parametrize("b,hq,hkv,max_s,ctx,d,splits", [
    (2, 16, 8, 512, 300, 128, 0), (3, 4, 4, 256, 256, 128, 1), (1, 8, 2, 1024, 1, 128, 4), (4, 16, 8, 2320, 2049, 128, 0),
    (2, 12, 12, 640, 129, 64, 3), (1, 32, 8, 384, 128, 128, 8), (2, 2, 1, 128, 77, 64, 0)])
def test_decode_attention_contiguous_cache(backend, oracle, b, hq, hkv, max_s, ctx, d, splits):
    run_case(oracle, b, hq, hkv, max_s, ctx, d, splits)


def test_decode_attention_over_no_keys_gives_zero_rows(backend):
    """A context length of 0 can only arrive from device memory (the host argument is range-checked).
    Attention over no key is defined as a zero row, with one split (the kernel stores directly) and
    with several (the combine kernel stores): `out` never keeps its previous contents."""
    b, hq, hkv, max_s, d = 2, 8, 4, 256, 128
    q = lib.round_to_bf16(synth.normal("q", (b, hq, 1, d)))
    kc = lib.round_to_bf16(synth.normal("kc", (b, hkv, max_s, d)))
    for splits in (1, 3, 0):
        got = _decode(q, kc, kc, 0, splits, ctx_on_device=True)
        assert np.array_equal(got, np.zeros_like(got)), f"splits={splits}"


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
