"""CPU tests of the oracle against independent float64 / torch-CPU evaluations.

The reference ships no golden vectors for this path, so these are the pins the oracle has: each
restated operator is compared with a float64 formulation written independently here (and with
torch on CPU where the reference's semantics coincide with PyTorch's), and each deliberate
deviation of the reference from PyTorch is asserted explicitly.
"""
import math

import numpy as np
import pytest
import torch

from kandle_b200 import synth


def test_gemm_nt_matches_float64(oracle):
    x = synth.normal("x", (37, 129))
    w = synth.normal("w", (53, 129))
    y = oracle.linear(x, w)
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()


def test_linear_bias_is_separate_add(oracle):
    x, w, b = synth.normal("x", (5, 16)), synth.normal("w", (8, 16)), synth.normal("b", (8,))
    y = oracle.linear(x, w, b)
    assert np.array_equal(y, (oracle.linear(x, w) + b).astype(np.float32))


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
def test_matmul4d_strided_views(oracle, trans_a, trans_b):
    a = synth.normal("a", (2, 3, 5, 7))
    b = synth.normal("b", (3, 7, 4))
    av = np.ascontiguousarray(a.transpose(0, 1, 3, 2)) if trans_a else a
    bv = np.ascontiguousarray(b.transpose(0, 2, 1)) if trans_b else b
    c = synth.normal("c", (2, 3, 5, 4))
    y = oracle.matmul4d(av, bv, trans_a=trans_a, trans_b=trans_b, alpha=0.5, beta=2.0, c=c)
    ref = 0.5 * (a.astype(np.float64) @ b.astype(np.float64)) + 2.0 * c
    assert np.abs(y - ref).max() < 1e-5
    # a non-contiguous view (transposed without copying) must read through its strides
    y2 = oracle.matmul4d(a, np.ascontiguousarray(b.transpose(0, 2, 1)).transpose(0, 2, 1))
    assert np.abs(y2 - a @ b).max() < 1e-5


def test_sdpa_tile_config_follows_16kb_rule(oracle):
    assert oracle.sdpa_tile_config(128, 128, 128) == (8, 4)
    assert oracle.sdpa_tile_config(64, 1500, 1500) == (16, 8)
    assert oracle.sdpa_tile_config(128, 1, 700) == (1, 4)    # chosen before clamping to Sq


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("hq,hkv,sq,skv,d", [(16, 8, 128, 128, 128), (4, 4, 33, 33, 64), (8, 2, 1, 77, 128), (2, 1, 17, 40, 32)])
def test_sdpa_matches_float64(oracle, causal, hq, hkv, sq, skv, d):
    q, k, v = synth.normal("q", (2, hq, sq, d)), synth.normal("k", (2, hkv, skv, d)), synth.normal("v", (2, hkv, skv, d))
    o = oracle.sdpa(q, k, v, is_causal=causal)
    r = hq // hkv
    kk, vv = np.repeat(k, r, 1).astype(np.float64), np.repeat(v, r, 1).astype(np.float64)
    s = (q.astype(np.float64) @ kk.transpose(0, 1, 3, 2)) / math.sqrt(d)
    if causal:  # top-left aligned: column > row is masked, whatever Skv - Sq is
        s = np.where(np.arange(skv)[None, :] > np.arange(sq)[:, None], -np.inf, s)
    p = np.exp(s - s.max(-1, keepdims=True))
    ref = (p / p.sum(-1, keepdims=True)) @ vv
    assert np.abs(o - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())


def test_sdpa_equals_torch_when_semantics_coincide(oracle):
    q, k, v = synth.normal("q", (1, 4, 50, 64)), synth.normal("k", (1, 4, 50, 64)), synth.normal("v", (1, 4, 50, 64))
    for causal in (False, True):
        ref = torch.nn.functional.scaled_dot_product_attention(torch.tensor(q), torch.tensor(k), torch.tensor(v),
                                                               is_causal=causal).numpy()
        assert np.abs(oracle.sdpa(q, k, v, is_causal=causal) - ref).max() < 2e-6


def test_sdpa_block_size_only_changes_rounding(oracle):
    q, k, v = synth.normal("q", (1, 2, 40, 128)), synth.normal("k", (1, 2, 40, 128)), synth.normal("v", (1, 2, 40, 128))
    a = oracle.sdpa(q, k, v, is_causal=True)
    b = oracle.sdpa(q, k, v, is_causal=True, block_kv=32)
    assert np.abs(a - b).max() < 1e-5


def test_sdpa_3d_means_batch_one(oracle):
    q, k, v = synth.normal("q", (6, 20, 64)), synth.normal("k", (6, 20, 64)), synth.normal("v", (6, 20, 64))
    assert np.array_equal(oracle.sdpa(q, k, v), oracle.sdpa(q[None], k[None], v[None])[0])


def test_rms_norm_formula(oracle):
    x, w = synth.normal("x", (7, 128)), synth.normal("w", (128,), 0.1, 1.0)
    y = oracle.rms_norm(x, w, 1e-6)
    xd = x.astype(np.float64)
    ref = xd * (1.0 / np.sqrt((xd ** 2).mean(-1, keepdims=True) + 1e-6)) * w
    assert np.abs(y - ref).max() < 1e-5
    t = torch.nn.functional.rms_norm(torch.tensor(x), (128,), torch.tensor(w), 1e-6).numpy()
    assert np.abs(y - t).max() < 1e-5


def test_layer_norm_biased_variance(oracle):
    x, w, b = synth.normal("x", (5, 768), 3.0, 0.7), synth.normal("w", (768,), 0.1, 1.0), synth.normal("b", (768,))
    y = oracle.layer_norm(x, w, b, 1e-5)
    t = torch.nn.functional.layer_norm(torch.tensor(x).double(), (768,), torch.tensor(w).double(),
                                       torch.tensor(b).double(), 1e-5).numpy()
    assert np.abs(y - t).max() < 2e-5


def test_softmax(oracle):
    x = synth.normal("x", (9, 333), 4.0)
    t = torch.softmax(torch.tensor(x).double(), -1).numpy()
    assert np.abs(oracle.softmax(x) - t).max() < 1e-6


def test_gelu_is_always_tanh_form_with_clamp(oracle):
    x = np.linspace(-30, 30, 2001, dtype=np.float32)
    y = oracle.unary("gelu", x)
    t = torch.nn.functional.gelu(torch.tensor(x).double(), approximate="tanh").numpy()
    assert np.abs(y - t).max() < 1e-5
    exact = torch.nn.functional.gelu(torch.tensor(x).double()).numpy()
    assert np.abs(y - exact).max() > 1e-4          # it is NOT the erf form
    assert np.isfinite(y).all()


def test_silu_clamps_its_exponent(oracle):
    x = np.array([-1000.0, -88.0, -1.0, 0.0, 1.0, 88.0, 1000.0], dtype=np.float32)
    y = oracle.unary("silu", x)
    assert np.isfinite(y).all()
    assert y[-1] == np.float32(1000.0) and abs(y[0]) < 1e-30
    mid = x[1:-1].astype(np.float64)
    assert np.abs(y[1:-1] - mid / (1 + np.exp(-mid))).max() < 1e-5


def test_rope_half_split_layout(oracle):
    inv = oracle.rope_inv_freq(128, 1e6)
    assert inv.dtype == np.float32 and inv[0] == 1.0
    assert abs(float(inv[32]) - 1e6 ** (-0.5)) < 1e-9
    cos, sin = oracle.rope_tables(np.arange(5, 9, dtype=np.int32), 128, 1e6)
    assert cos.shape == (4, 128) and np.array_equal(cos[:, :64], cos[:, 64:])
    x = synth.normal("x", (1, 2, 4, 128))
    y = oracle.apply_rope(x, cos, sin)
    x1, x2 = x[..., :64].astype(np.float64), x[..., 64:].astype(np.float64)
    c, s = cos[:, :64].astype(np.float64), sin[:, :64].astype(np.float64)
    ref = np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    assert np.abs(y - ref).max() < 1e-6


def test_embedding_and_argmax(oracle):
    w = synth.normal("e", (50, 8))
    ids = np.array([[0, 49, 7], [7, 7, 1]], dtype=np.int32)
    assert np.array_equal(oracle.embedding(w, ids), w[ids])
    with pytest.raises(IndexError):
        oracle.embedding(w, np.array([50], dtype=np.int32))
    x = synth.normal("x", (4, 1000))
    x[2, 10] = x[2, 900] = 99.0                      # ties resolve to the lowest index
    assert np.array_equal(oracle.argmax_rows(x), np.argmax(x, -1).astype(np.int32))
    assert oracle.argmax_rows(x)[2] == 10


def test_conv1d_im2col(oracle):
    x, w, b = synth.normal("x", (2, 5, 31)), synth.normal("w", (7, 5, 3)), synth.normal("b", (7,))
    for stride in (1, 2):
        y = oracle.conv1d(x, w, b, stride, 1)
        t = torch.nn.functional.conv1d(torch.tensor(x).double(), torch.tensor(w).double(), torch.tensor(b).double(),
                                       stride=stride, padding=1).numpy()
        assert y.shape == t.shape and np.abs(y - t).max() < 1e-5


def _tiny_qwen3(oracle):
    cfg = oracle.Qwen3Config(vocab_size=97, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=32)
    w = synth.qwen3_weights(vocab=97, hidden=64, inter=96, layers=2, heads=4, kv_heads=2, head_dim=32, std=0.1,
                            norm_jitter=0.05)
    return cfg, w


def test_qwen3_oracle_matches_independent_torch_model(oracle):
    """The whole operator sequence against a from-scratch float64 torch implementation."""
    cfg, w = _tiny_qwen3(oracle)
    ids = synth.token_ids("ids", (2, 11), 97)
    got = oracle.Qwen3Oracle(cfg, w).logits(ids)
    W = {k: torch.tensor(v).double() for k, v in w.items()}

    def rms(x, g):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + cfg.rms_norm_eps) * g

    B, S = ids.shape
    h = W["model.embed_tokens.weight"][torch.tensor(ids).long()]
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, 16).double() / 16))
    ang = torch.arange(S).double()[:, None] * inv[None]
    cos, sin = torch.cat([ang.cos()] * 2, -1), torch.cat([ang.sin()] * 2, -1)

    def rope(x):
        return x * cos + torch.cat([-x[..., 16:], x[..., :16]], -1) * sin

    for i in range(2):
        p = f"model.layers.{i}."
        x = rms(h, W[p + "input_layernorm.weight"])
        q = (x @ W[p + "self_attn.q_proj.weight"].T).view(B, S, 4, 32)
        k = (x @ W[p + "self_attn.k_proj.weight"].T).view(B, S, 2, 32)
        v = (x @ W[p + "self_attn.v_proj.weight"].T).view(B, S, 2, 32)
        q, k = rms(q, W[p + "self_attn.q_norm.weight"]), rms(k, W[p + "self_attn.k_norm.weight"])
        q, k, v = rope(q.transpose(1, 2)), rope(k.transpose(1, 2)), v.transpose(1, 2)
        o = torch.nn.functional.scaled_dot_product_attention(q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1),
                                                             is_causal=True)
        h = h + o.transpose(1, 2).reshape(B, S, 128) @ W[p + "self_attn.o_proj.weight"].T
        x = rms(h, W[p + "post_attention_layernorm.weight"])
        h = h + (torch.nn.functional.silu(x @ W[p + "mlp.gate_proj.weight"].T) * (x @ W[p + "mlp.up_proj.weight"].T)) \
            @ W[p + "mlp.down_proj.weight"].T
    ref = (rms(h, W["model.norm.weight"]) @ W["model.embed_tokens.weight"].T).numpy()
    assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()


def test_qwen3_kv_cache_decode_equals_full_forward(oracle):
    """Prefill + cached single-token steps must reproduce a full re-forward (the reference's two
    generation paths agree the same way)."""
    cfg, w = _tiny_qwen3(oracle)
    m = oracle.Qwen3Oracle(cfg, w)
    ids = synth.token_ids("ids", (2, 9), 97)
    full = m.logits(ids)
    cache = oracle.StaticKVCacheOracle(cfg, 2, 16)
    pre = m.logits(ids[:, :6], cache, 0)
    assert np.abs(pre - full[:, :6]).max() < 1e-5
    for t in range(6, 9):
        step = m.logits(ids[:, t:t + 1], cache, t)
        assert np.abs(step[:, 0] - full[:, t]).max() < 1e-5
    toks = m.greedy_generate(ids, 4)
    assert toks.shape == (2, 4) and toks.dtype == np.int32


def test_whisper_encoder_oracle_shapes_and_torch_block(oracle):
    cfg = oracle.WhisperEncoderConfig(n_mels=8, n_audio_ctx=20, n_audio_state=32, n_audio_head=4, n_audio_layer=1)
    w = synth.whisper_encoder_weights(n_mels=8, state=32, layers=1, n_ctx=20, std=0.1)
    mel = synth.normal("mel", (2, 8, 40))
    y = oracle.WhisperEncoderOracle(cfg, w).forward(mel)
    assert y.shape == (2, 20, 32)
    W = {k: torch.tensor(v).double() for k, v in w.items()}
    F = torch.nn.functional
    x = F.gelu(F.conv1d(torch.tensor(mel).double(), W["conv1.weight"], W["conv1.bias"], padding=1), approximate="tanh")
    x = F.gelu(F.conv1d(x, W["conv2.weight"], W["conv2.bias"], stride=2, padding=1), approximate="tanh")
    x = x.permute(0, 2, 1) + W["embed_positions.weight"][:20]
    p = "layers.0."
    mha = torch.nn.MultiheadAttention(32, 4, batch_first=True).double()
    mha.in_proj_weight.data, mha.in_proj_bias.data = W[p + "self_attn.in_proj_weight"], W[p + "self_attn.in_proj_bias"]
    mha.out_proj.weight.data, mha.out_proj.bias.data = W[p + "self_attn.out_proj.weight"], W[p + "self_attn.out_proj.bias"]
    yl = F.layer_norm(x, (32,), W[p + "self_attn_layer_norm.weight"], W[p + "self_attn_layer_norm.bias"])
    x = x + mha(yl, yl, yl, need_weights=False)[0]
    yl = F.layer_norm(x, (32,), W[p + "final_layer_norm.weight"], W[p + "final_layer_norm.bias"])
    x = x + F.gelu(yl @ W[p + "fc1.weight"].T + W[p + "fc1.bias"], approximate="tanh") @ W[p + "fc2.weight"].T + W[p + "fc2.bias"]
    ref = F.layer_norm(x, (32,), W["layer_norm.weight"], W["layer_norm.bias"]).detach().numpy()
    assert np.abs(y - ref).max() < 1e-4


def test_sampler_restatement_against_a_sorted_float64_formulation(oracle):
    """oracle.sample restates the reference's host sampler; here the same selection is written the
    textbook way (sort, cumulative sums in float64) and the kept sets / draws must agree."""
    rng = np.random.default_rng(5)
    lg = (rng.standard_normal(3000) * 2.5).astype(np.float32)
    for temperature, top_k, top_p in [(1.0, 0, 1.0), (0.7, 50, 1.0), (1.0, 0, 0.9), (0.8, 40, 0.95), (1.3, 5, 0.5)]:
        x = lg.astype(np.float64) / temperature
        p = np.exp(x - x.max())
        p /= p.sum()
        order = np.argsort(-lg.astype(np.float64), kind="stable")
        keep = len(lg)
        if 0 < top_k < len(lg):
            keep = top_k
        if top_p < 1.0:
            cum = np.cumsum(p[order[:keep]])
            keep = min(keep, int(np.searchsorted(cum, top_p, side="left")) + 1)
        kept = np.zeros(len(lg), bool)
        kept[order[:keep]] = True
        q = np.where(kept, p, 0.0)
        q /= q.sum()
        for r in (0.01, 0.25, 0.5, 0.75, 0.99):
            got = oracle.sample(lg, temperature, top_k, top_p, True, r)
            assert np.array_equal(got["probs"] > 0, kept)
            assert np.abs(got["probs"] - q).max() <= 1e-6
            assert got["token"] == int(np.searchsorted(np.cumsum(q), r, side="right"))
    g = oracle.sample(lg, 0.7, 0, 1.0, False)
    assert g["token"] == int(lg.argmax())
    tied = np.array([1.0, 3.0, 3.0, -1.0, 3.0], np.float32)
    assert oracle.sample(tied, 1.0, 2, 1.0, True, 0.99)["token"] == 2        # stable sort keeps indices 1 and 2
    assert oracle.sample(tied, 1.0, 0, 1.0, False)["token"] == 1


def test_log_mel_restatement_against_torch_stft(oracle):
    """oracle.whisper_log_mel against the same pipeline written with torch.stft (constant-mode centre
    padding, the symmetric Hann window and the slaney filterbank the reference builds)."""
    from kandle_b200 import audio
    w = audio.hann_window_host(400)
    fb = audio.melscale_fbanks_host(201, 0, 8000, 80, 16000, "slaney", "slaney")
    assert abs(w[0]) == 0.0 and abs(w[399]) < 1e-7 and abs(w[200] - w[199]) < 1e-6      # symmetric: M = N - 1
    assert fb.shape == (201, 80) and (fb >= 0).all() and ((fb > 0).sum(0) >= 1).all()
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(16000 * 3) * 0.1).astype(np.float32)
    got = oracle.whisper_log_mel(x, w, fb)
    xt = torch.zeros(480000)
    xt[: x.size] = torch.from_numpy(x)
    st = torch.stft(xt, 400, 160, window=torch.from_numpy(w), center=True, pad_mode="constant", return_complex=True)
    mel = (torch.from_numpy(fb).T @ (st.abs() ** 2))[:, :3000]
    ls = torch.clamp(mel, min=1e-10).log10()
    ls = (torch.maximum(ls, ls.max() - 8.0) + 4.0) / 4.0
    assert got.shape == (1, 80, 3000)
    assert np.abs(ls.numpy() - got[0]).max() <= 5e-6


def test_whisper_decoder_restatement_against_float64(oracle):
    """WhisperDecoderOracle against a direct float64 evaluation of the same block structure."""
    from kandle_b200 import synth as sy
    V, E, H, L, C = 61, 32, 4, 2, 16
    w = sy.whisper_decoder_weights(vocab=V, state=E, layers=L, n_ctx=C, std=0.1)
    cfg = oracle.WhisperDecoderConfig(n_vocab=V, n_text_ctx=C, n_text_state=E, n_text_head=H, n_text_layer=L)
    tokens = sy.token_ids("dec-cpu", (2, 7), V)
    xa = sy.normal("dec-cpu-xa", (2, 11, E), 0.5)
    got = oracle.WhisperDecoderOracle(cfg, w).forward(tokens, xa, offset=3)
    W = {k: v.astype(np.float64) for k, v in w.items()}

    def ln(x, p):
        m = x.mean(-1, keepdims=True)
        v = ((x - m) ** 2).mean(-1, keepdims=True)
        return (x - m) / np.sqrt(v + 1e-5) * W[p + ".weight"] + W[p + ".bias"]

    def mha(p, xq, xkv, causal):
        Wi, bi = W[p + ".in_proj_weight"], W[p + ".in_proj_bias"]
        q, k, v = xq @ Wi[:E].T + bi[:E], xkv @ Wi[E:2 * E].T + bi[E:2 * E], xkv @ Wi[2 * E:].T + bi[2 * E:]
        B, Lq, S, D = xq.shape[0], xq.shape[1], xkv.shape[1], E // H
        q, k, v = (t.reshape(B, -1, H, D).transpose(0, 2, 1, 3) for t in (q, k, v))
        s = q @ k.transpose(0, 1, 3, 2) / math.sqrt(D)
        if causal:
            s = s + np.where(np.arange(S)[None, :] > np.arange(Lq)[:, None], -np.inf, 0.0)
        s = np.exp(s - s.max(-1, keepdims=True))
        o = (s / s.sum(-1, keepdims=True)) @ v
        return o.transpose(0, 2, 1, 3).reshape(B, Lq, E) @ W[p + ".out_proj.weight"].T + W[p + ".out_proj.bias"]

    def gelu(x):   # tanh form with the reference's clamp
        return 0.5 * x * (1.0 + np.tanh(np.clip(0.7978845608028654 * (x + 0.044715 * x ** 3), -20, 20)))

    x = W["embed_tokens.weight"][tokens] + W["embed_positions.weight"][3:10][None]
    for i in range(L):
        p = f"layers.{i}."
        x = x + mha(p + "self_attn", ln(x, p + "self_attn_layer_norm"), ln(x, p + "self_attn_layer_norm"), True)
        x = x + mha(p + "encoder_attn", ln(x, p + "encoder_attn_layer_norm"), xa.astype(np.float64), False)
        y = gelu(ln(x, p + "final_layer_norm") @ W[p + "fc1.weight"].T + W[p + "fc1.bias"])
        x = x + y @ W[p + "fc2.weight"].T + W[p + "fc2.bias"]
    ref = ln(x, "layer_norm") @ W["embed_tokens.weight"].T
    assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()


def test_mel_filterbank_against_an_independent_slaney_formulation():
    """melscale_fbanks_host (mirror of audio/functional/filterbank.ts:88-150) against the textbook
    construction of Slaney-scale, area-normalised triangular filters in float64."""
    from kandle_b200 import audio
    n_freqs, n_mels, sr, f_max = 201, 80, 16000, 8000.0
    fb = audio.melscale_fbanks_host(n_freqs, 0.0, f_max, n_mels, sr, "slaney", "slaney")

    def hz_to_mel(f):
        f = np.asarray(f, dtype=np.float64)
        lin = f / (200.0 / 3.0)
        log = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0)
        return np.where(f >= 1000.0, log, lin)

    def mel_to_hz(m):
        m = np.asarray(m, dtype=np.float64)
        return np.where(m >= 15.0, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3.0))

    edges = mel_to_hz(np.linspace(hz_to_mel(0.0), hz_to_mel(f_max), n_mels + 2))
    freqs = np.linspace(0.0, sr / 2, n_freqs)
    lower = (freqs[:, None] - edges[None, :-2]) / (edges[1:-1] - edges[:-2])[None, :]
    upper = (edges[None, 2:] - freqs[:, None]) / (edges[2:] - edges[1:-1])[None, :]
    ref = np.maximum(0.0, np.minimum(lower, upper)) * (2.0 / (edges[2:] - edges[:-2]))[None, :]
    assert fb.shape == ref.shape == (n_freqs, n_mels)
    assert np.abs(fb - ref).max() <= 2e-6 * ref.max()          # the reference stores band edges in float32
    w = audio.hann_window_host(400, periodic=True)
    assert abs(w[200] - 1.0) < 1e-7 and abs(w[1] - w[399]) < 1e-7      # periodic form: w[n] = w[N - n]
    basis = audio.dft_basis_host(400)
    x = np.random.default_rng(3).standard_normal(400)
    spec = np.fft.rfft(x)
    got = x @ basis.astype(np.float64)
    assert np.abs(got[:201] - spec.real).max() <= 1e-4 and np.abs(got[201:] - spec.imag).max() <= 1e-4


def test_philox4x32_10_known_answer_vectors():
    """The generator under the reference's `randn` key is Philox4x32-10; its authors' known-answer
    vectors (Random123 kat_vectors, philox4x32 with 10 rounds) pin the restatement bit for bit."""
    from oracle import oracle as orc
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0), (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, want in kat:
        got = orc.philox4x32_10(np.array([ctr], np.uint32), key[0], key[1])[0]
        assert tuple(int(x) for x in got) == want


def test_randn_stream_is_normal_and_windows_agree():
    from oracle import oracle as orc
    z = orc.randn(400000, 77, base_offset=5)
    assert abs(float(z.mean())) < 5e-3 and abs(float(z.std()) - 1.0) < 5e-3
    assert abs(float((z ** 3).mean())) < 2e-2 and abs(float((z ** 4).mean()) - 3.0) < 5e-2
    # a window of the stream equals the same elements of the whole stream; the offset shifts pairs
    assert np.array_equal(orc.randn(1000, 77, base_offset=5, first=1235), z[1235:2235])
    assert np.array_equal(orc.randn(1000, 77, base_offset=6), z[2:1002])
