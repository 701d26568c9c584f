"""GPU parity of the fused bf16 kernels (skinny GEMM with split-K partials, q/k-norm + RoPE + cache
write, SiLU*up, residual + RMSNorm, RoPE tables) against the oracle's unfused operator sequence."""
import ctypes

import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


_KEEP = []   # temporaries must outlive the enqueue call: a dropped Tensor releases its storage


@pytest.fixture(autouse=True)
def _clear_keep():
    yield
    _KEEP.clear()


def bf(a):
    t = Tensor(a, dtype="bfloat16")
    _KEEP.append(t)
    return t


def f32(a):
    t = Tensor(a)
    _KEEP.append(t)
    return t


def close_bf16(got, ref, extra=2e-3):
    ref = ref.astype(np.float64)
    err = np.abs(got - ref)
    assert (err <= np.abs(ref) * 2.0 ** -7 + extra * np.abs(ref).max()).all(), f"worst {err.max():.3e}"


@pytest.mark.parametrize("m,n,k,splits", [(1, 256, 128, 1), (32, 4096, 1024, 0), (32, 1024, 3072, 6), (7, 1000, 264, 2),
                                          (128, 384, 512, 4), (33, 152064, 256, 1), (100, 130, 64, 1)])
def test_skinny_gemm_partials_sum_to_the_product(backend, oracle, m, n, k, splits):
    x, w = lib.round_to_bf16(synth.normal("x", (m, k))), lib.round_to_bf16(synth.normal("w", (n, k), 0.05))
    ref = oracle.linear(x, w)
    if splits == 0:
        s = ctypes.c_int(0)
        lib.call("kd_linear_bf16_skinny_splits", ctypes.c_int64(n), ctypes.c_int64(k), ctypes.byref(s))
        splits = s.value
        assert 1 <= splits <= max(1, k // 64)
    out = core.empty((splits, m, n), "float32")
    lib.call("kd_linear_bf16_skinny", _r(bf(x)), _r(bf(w)), 0, _r(out))
    got = out.dataAsync().sum(0)
    assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()
    if splits == 1:
        ob = core.empty((m, n), "bfloat16")
        lib.call("kd_linear_bf16_skinny", _r(bf(x)), _r(bf(w)), 0, _r(ob))
        close_bf16(ob.dataAsync(), ref)


def test_skinny_gemm_swiglu_epilogue(backend, oracle):
    m, K, I = 32, 1024, 3072
    x = lib.round_to_bf16(synth.normal("x", (m, K)))
    wg, wu = lib.round_to_bf16(synth.normal("wg", (I, K), 0.03)), lib.round_to_bf16(synth.normal("wu", (I, K), 0.03))
    fused = np.stack([wg.reshape(I // 16, 16, K), wu.reshape(I // 16, 16, K)], 1).reshape(2 * I, K)
    out = core.empty((m, I), "bfloat16")
    lib.call("kd_linear_bf16_skinny", _r(bf(x)), _r(bf(fused)), 2, _r(out))
    close_bf16(out.dataAsync(), oracle.mul(oracle.unary("silu", oracle.linear(x, wg)), oracle.linear(x, wu)))


def test_rope_table_matches_oracle(backend, oracle):
    inv = oracle.rope_inv_freq(128, 1e6)
    cos, sin = core.empty((40, 64), "float32"), core.empty((40, 64), "float32")
    lib.call("kd_rope_table", _r(f32(inv)), None, 2000, 40, _r(cos), _r(sin))
    rc, rs = oracle.rope_tables(np.arange(2000, 2040, dtype=np.int32), 128, 1e6)
    assert np.abs(cos.dataAsync() - rc[:, :64]).max() < 1e-6 and np.abs(sin.dataAsync() - rs[:, :64]).max() < 1e-6
    pos = Tensor(np.array([77], np.int32))
    c1, s1 = core.empty((1, 64), "float32"), core.empty((1, 64), "float32")
    lib.call("kd_rope_table", _r(f32(inv)), _r(pos), 0, 1, _r(c1), _r(s1))
    assert np.abs(c1.dataAsync() - oracle.rope_tables(np.array([77], np.int32), 128, 1e6)[0][:, :64]).max() < 1e-6


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("partials", [0, 3])
def test_qkv_norm_rope_cachewrite(backend, oracle, d, partials):
    B, S, Hq, Hkv, max_s, pos0 = 2, 5, 4, 2, 16, 3
    n = (Hq + 2 * Hkv) * d
    qkv = lib.round_to_bf16(synth.normal("qkv", (B, S, n)))
    qw, kw = lib.round_to_bf16(synth.normal("qw", (d,), 0.1, 1.0)), lib.round_to_bf16(synth.normal("kw", (d,), 0.1, 1.0))
    inv = oracle.rope_inv_freq(d, 1e6)
    cos_t, sin_t = core.empty((S, d // 2), "float32"), core.empty((S, d // 2), "float32")
    lib.call("kd_rope_table", _r(f32(inv)), None, pos0, S, _r(cos_t), _r(sin_t))
    kc, vc = core.zeros((B, Hkv, max_s, d), "bfloat16"), core.zeros((B, Hkv, max_s, d), "bfloat16")
    q_out = core.empty((B, S, Hq, d), "bfloat16")
    if partials:
        parts = synth.normal("parts", (partials - 1, B * S, n), 0.3)
        last = qkv.reshape(B * S, n) - parts.sum(0)
        src = Tensor(np.concatenate([parts, last[None]], 0).astype(np.float32))
        qkv_eff = (parts.sum(0, dtype=np.float32) + last.astype(np.float32)).reshape(B, S, n)
    else:
        src, qkv_eff = bf(qkv), qkv
    lib.call("kd_qkv_norm_rope_cachewrite", _r(src), _r(bf(qw)), _r(bf(kw)), ctypes.c_float(1e-6), _r(cos_t), _r(sin_t), _r(kc),
             _r(vc), None, pos0, _r(q_out))
    # oracle: the unfused sequence
    q = qkv_eff[..., :Hq * d].reshape(B, S, Hq, d)
    k = qkv_eff[..., Hq * d:(Hq + Hkv) * d].reshape(B, S, Hkv, d)
    v = qkv_eff[..., (Hq + Hkv) * d:].reshape(B, S, Hkv, d)
    cos, sin = oracle.rope_tables(np.arange(pos0, pos0 + S, dtype=np.int32), d, 1e6)
    qr = oracle.apply_rope(oracle.rms_norm(q, qw, 1e-6).transpose(0, 2, 1, 3), cos, sin)
    kr = oracle.apply_rope(oracle.rms_norm(k, kw, 1e-6).transpose(0, 2, 1, 3), cos, sin)
    close_bf16(q_out.dataAsync(), qr.transpose(0, 2, 1, 3), 4e-3)
    kref = np.zeros((B, Hkv, max_s, d), np.float32)
    vref = np.zeros((B, Hkv, max_s, d), np.float32)
    kref[:, :, pos0:pos0 + S] = kr
    vref[:, :, pos0:pos0 + S] = v.transpose(0, 2, 1, 3)
    close_bf16(kc.dataAsync(), kref, 4e-3)
    close_bf16(vc.dataAsync(), vref, 4e-3)


def test_qkv_cachewrite_overflow_is_reported(backend):
    kc = core.zeros((1, 1, 4, 64), "bfloat16")
    q_out = core.empty((1, 2, 1, 64), "bfloat16")
    zt = core.zeros((2, 32), "float32")
    args = lambda start: (_r(bf(np.zeros((1, 2, 192), np.float32))), _r(bf(np.ones(64, np.float32))), _r(bf(np.ones(64, np.float32))),
                          ctypes.c_float(1e-6), _r(zt), _r(zt), _r(kc), _r(kc),
                          None, start, _r(q_out))
    with pytest.raises(lib.KandleCudaError) as e:
        lib.call("kd_qkv_norm_rope_cachewrite", *args(3))
    assert "Cache overflow" in str(e.value)
    # a device-side position cannot be checked on the host: the kernel refuses the write and flags it
    pos = Tensor(np.array([3], np.int32))
    lib.call("kd_qkv_norm_rope_cachewrite", *(args(0)[:8] + (_r(pos), 0, _r(q_out))))
    with pytest.raises(lib.KandleCudaError) as e:
        backend.synchronize()
    assert e.value.status == 6
    backend.synchronize()


@pytest.mark.parametrize("partials", [0, 4])
def test_swiglu(backend, oracle, partials):
    rows, inter = 9, 96
    g, u = synth.normal("g", (rows, inter), 2.0), synth.normal("u", (rows, inter))
    fused = np.stack([g.reshape(rows, inter // 16, 16), u.reshape(rows, inter // 16, 16)], 2).reshape(rows, 2 * inter)
    out = core.empty((rows, inter), "bfloat16")
    if partials:
        parts = synth.normal("p", (partials - 1, rows, 2 * inter), 0.5)
        src = Tensor(np.concatenate([parts, (fused - parts.sum(0))[None]], 0).astype(np.float32))
        eff = src.dataAsync().sum(0)
        g = eff.reshape(rows, inter // 16, 2, 16)[:, :, 0].reshape(rows, inter)
        u = eff.reshape(rows, inter // 16, 2, 16)[:, :, 1].reshape(rows, inter)
    else:
        fused = lib.round_to_bf16(fused)
        g = fused.reshape(rows, inter // 16, 2, 16)[:, :, 0].reshape(rows, inter)
        u = fused.reshape(rows, inter // 16, 2, 16)[:, :, 1].reshape(rows, inter)
        src = bf(fused)
    lib.call("kd_swiglu", _r(src), _r(out))
    close_bf16(out.dataAsync(), oracle.mul(oracle.unary("silu", g), u))


@pytest.mark.parametrize("rows", [5, 1500])
@pytest.mark.parametrize("n", [1024, 2560, 64])
@pytest.mark.parametrize("mode", ["plain", "residual", "partials"])
def test_add_rmsnorm(backend, oracle, n, mode, rows):
    x, r, w = synth.normal("x", (rows, n)), lib.round_to_bf16(synth.normal("r", (rows, n))), lib.round_to_bf16(synth.normal("w", (n,), 0.1, 1.0))
    norm, summ = core.empty((rows, n), "bfloat16"), core.empty((rows, n), "bfloat16")
    if mode == "plain":
        xb = lib.round_to_bf16(x)
        lib.call("kd_add_rmsnorm", _r(bf(xb)), None, _r(bf(w)), ctypes.c_float(1e-6), None, _r(norm))
        close_bf16(norm.dataAsync(), oracle.rms_norm(xb, w, 1e-6))
        return
    if mode == "residual":
        xb = lib.round_to_bf16(x)
        src, total = bf(xb), xb + r
    else:
        parts = synth.normal("p", (3 if rows < 1000 else 1, rows, n), 0.4)   # the many-row kernel takes one fp32 slice
        src, total = Tensor(parts), parts.sum(0, dtype=np.float32) + r
    lib.call("kd_add_rmsnorm", _r(src), _r(bf(r)), _r(bf(w)), ctypes.c_float(1e-6), _r(summ), _r(norm))
    t = lib.round_to_bf16(total.astype(np.float32))
    got_sum = summ.dataAsync()
    close_bf16(got_sum, total)
    close_bf16(norm.dataAsync(), oracle.rms_norm(got_sum, w, 1e-6))     # the norm is taken of the rounded sum


def test_graph_capture_replays_with_device_side_state(backend):
    """A captured increment is replayed; the launch counter counts replayed nodes."""
    s = Tensor(np.array([5], np.int32))
    lib.call("kd_increment_i32", _r(s), 1)
    lib.call("kd_graph_begin")
    lib.call("kd_increment_i32", _r(s), 2)
    lib.call("kd_increment_i32", _r(s), 3)
    g = ctypes.c_uint64(0)
    lib.call("kd_graph_end", ctypes.byref(g))
    assert s.dataAsync()[0] == 6                      # capturing did not execute anything
    n0 = backend.launch_count()
    for _ in range(3):
        lib.call("kd_graph_launch", g)
    assert s.dataAsync()[0] == 6 + 3 * 5 and backend.launch_count() - n0 >= 6
    lib.call("kd_graph_destroy", g)


def test_qkv_gemm_with_fused_norm_rope_cachewrite_matches_the_two_kernel_path(backend, oracle):
    """kd_qkv_linear_norm_rope_cachewrite == kd_linear_bf16 followed by kd_qkv_norm_rope_cachewrite,
    and both follow the oracle's unfused sequence."""
    B, S, Hq, Hkv, K, max_s, pos0 = 2, 150, 4, 2, 256, 192, 7
    d, n = 128, (4 + 2 * 2) * 128
    x = lib.round_to_bf16(synth.normal("x", (B * S, K)))
    w = lib.round_to_bf16(synth.normal("w", (n, K), 0.06))
    qw, kw = lib.round_to_bf16(synth.normal("qw", (d,), 0.1, 1.0)), lib.round_to_bf16(synth.normal("kw", (d,), 0.1, 1.0))
    cos_t, sin_t = core.empty((S, 64), "float32"), core.empty((S, 64), "float32")
    lib.call("kd_rope_table", _r(f32(oracle.rope_inv_freq(d, 1e6))), None, pos0, S, _r(cos_t), _r(sin_t))
    tx, tw, tqw, tkw = bf(x), bf(w), bf(qw), bf(kw)
    outs = []
    for fused in (True, False):
        kc, vc = core.zeros((B, Hkv, max_s, d), "bfloat16"), core.zeros((B, Hkv, max_s, d), "bfloat16")
        q_out = core.empty((B, S, Hq, d), "bfloat16")
        if fused:
            lib.call("kd_qkv_linear_norm_rope_cachewrite", _r(tx), _r(tw), _r(tqw), _r(tkw), ctypes.c_float(1e-6), _r(cos_t), _r(sin_t),
                     _r(kc), _r(vc), pos0, _r(q_out))
        else:
            qkv = core.empty((B, S, n), "bfloat16")
            lib.call("kd_linear_bf16", _r(tx), _r(tw), None, 0, _r(qkv))
            lib.call("kd_qkv_norm_rope_cachewrite", _r(qkv), _r(tqw), _r(tkw), ctypes.c_float(1e-6), _r(cos_t), _r(sin_t), _r(kc), _r(vc),
                     None, pos0, _r(q_out))
        outs.append((q_out.dataAsync(), kc.dataAsync(), vc.dataAsync()))
    qkv_ref = oracle.linear(x, w).reshape(B, S, n)
    cos, sin = oracle.rope_tables(np.arange(pos0, pos0 + S, dtype=np.int32), d, 1e6)
    q = oracle.apply_rope(oracle.rms_norm(qkv_ref[..., :Hq * d].reshape(B, S, Hq, d), qw, 1e-6).transpose(0, 2, 1, 3), cos, sin)
    k = oracle.apply_rope(oracle.rms_norm(qkv_ref[..., Hq * d:(Hq + Hkv) * d].reshape(B, S, Hkv, d), kw, 1e-6).transpose(0, 2, 1, 3), cos, sin)
    v = qkv_ref[..., (Hq + Hkv) * d:].reshape(B, S, Hkv, d).transpose(0, 2, 1, 3)
    for q_got, k_got, v_got in outs:
        close_bf16(q_got, q.transpose(0, 2, 1, 3), 6e-3)
        close_bf16(k_got[:, :, pos0:pos0 + S], k, 6e-3)
        close_bf16(v_got[:, :, pos0:pos0 + S], v, 6e-3)
        assert not k_got[:, :, :pos0].any() and not k_got[:, :, pos0 + S:].any()      # nothing written outside [pos0, pos0+S)
    # the fused epilogue skips one bf16 rounding (of the projection), so the two paths agree to bf16 precision
    assert np.abs(outs[0][0] - outs[1][0]).max() <= 0.05 * np.abs(outs[1][0]).max()
