"""safetensors reader (mirror of packages/core/src/io/safetensor/*): header parsing and validation
on the CPU; upload of native bf16 bits and loading a module from a (sharded) checkpoint on the GPU."""
import json
import os
import struct

import numpy as np
import pytest

from kandle_b200 import io as kio
from kandle_b200 import lib, synth


def _write(path, header: dict, payload: bytes = b"", pad=True):
    hb = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        f.write(payload)


def test_round_trip_and_lazy_views(tmp_path):
    a = synth.normal("st.a", (5, 7))
    b = np.arange(12, dtype=np.int64).reshape(3, 4)
    c16 = lib.f32_to_bf16_bits(synth.normal("st.c", (4, 8)))
    p = str(tmp_path / "m.safetensors")
    kio.save_file({"a": a, "b": b, "c": (c16, "BF16"), "h": a.astype(np.float16)}, p, metadata={"format": "pt"})
    g = kio.loadSafetensor(p)
    assert not g.sharded and g.metadata == {"format": "pt"} and set(g.layers) == {"a", "b", "c", "h"}
    la, lc = g.getLayer("a"), g.getLayer("c")
    assert la.dtype == "float32" and la.shape == (5, 7) and la.numel == 35 and la.byteSize == 140
    assert np.array_equal(la.raw(), a) and np.array_equal(g.getLayer("b").raw(), b)
    assert lc.originalDtype == "BF16" and lc.dtype == "bfloat16"            # kept native, not widened
    assert np.array_equal(lc.raw(), c16)
    assert np.array_equal(lc.to_float32(), (c16.astype(np.uint32) << 16).view(np.float32))
    assert np.array_equal(g.getLayer("h").to_float32(), a.astype(np.float16).astype(np.float32))
    assert g.hasLayer("a") and not g.hasLayer("zz") and g.getLayer("zz") is None
    g.close()


def test_header_validation_matches_the_reference_messages(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(ValueError, match="too small"):
        kio.parseSafetensorFile(p)
    open(p, "wb").write(struct.pack("<II", 5, 1) + b"{}")
    with pytest.raises(ValueError, match="exceeds safe integer limit"):
        kio.parseSafetensorFile(p)
    open(p, "wb").write(struct.pack("<Q", 200 * 1024 * 1024))
    with pytest.raises(ValueError, match="exceeds safe limit"):
        kio.parseSafetensorFile(p)
    open(p, "wb").write(struct.pack("<Q", 0))
    with pytest.raises(ValueError, match="header size is 0"):
        kio.parseSafetensorFile(p)
    open(p, "wb").write(struct.pack("<Q", 50) + b"{}")
    with pytest.raises(ValueError, match="incomplete"):
        kio.parseSafetensorFile(p)
    open(p, "wb").write(struct.pack("<Q", 7) + b"{not js")
    with pytest.raises(ValueError, match="Invalid JSON"):
        kio.parseSafetensorFile(p)
    _write(p, {"w": {"dtype": "F8_E4M3", "shape": [2], "data_offsets": [0, 2]}}, b"\0\0")
    with pytest.raises(ValueError, match="Unsupported safetensors dtype: F8_E4M3"):
        kio.parseSafetensorFile(p)
    _write(p, {"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}, b"\0" * 12)
    with pytest.raises(ValueError, match="Data size mismatch for w: expected 16 bytes, got 12 bytes"):
        kio.parseSafetensorFile(p)
    _write(p, {"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}, b"\0" * 8)     # truncated payload
    with pytest.raises(ValueError, match="outside the file"):
        kio.parseSafetensorFile(p)
    _write(p, {"note": "not a tensor", "w": {"dtype": "U8", "shape": [0], "data_offsets": [0, 0]}})
    f = kio.parseSafetensorFile(p)
    assert set(f.layers) == {"w"} and f.layers["w"].numel == 0          # foreign entries are skipped, empty tensors allowed


def test_sharded_index(tmp_path):
    w = {f"layers.{i}.weight": synth.normal(f"sh.{i}", (3, 3)) for i in range(4)}
    kio.save_file({k: w[k] for k in list(w)[:2]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    kio.save_file({k: w[k] for k in list(w)[2:]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    idx = {"metadata": {"total_size": 144, "note": "x"},
           "weight_map": {k: ("model-00001-of-00002.safetensors" if i < 2 else "model-00002-of-00002.safetensors") for i, k in enumerate(w)}}
    ip = str(tmp_path / "model.safetensors.index.json")
    json.dump(idx, open(ip, "w"))
    g = kio.loadSafetensor(ip)
    assert g.sharded and g.totalSize == 144 and g.metadata == {"note": "x"} and len(g.files) == 2
    for k, v in w.items():
        assert np.array_equal(g.getLayer(k).raw(), v)
    idx["weight_map"]["ghost"] = "model-00002-of-00002.safetensors"
    json.dump(idx, open(ip, "w"))
    with pytest.raises(ValueError, match="Layer not found in shard model-00002-of-00002.safetensors: ghost"):
        kio.loadSafetensor(ip)
    idx["weight_map"]["ghost"] = "missing.safetensors"
    json.dump(idx, open(ip, "w"))
    with pytest.raises(ValueError, match="Shard file not found: missing.safetensors"):
        kio.loadSafetensor(ip)
    json.dump({"weights": {}}, open(ip, "w"))
    with pytest.raises(ValueError, match="weight_map must be an object"):
        kio.loadSafetensor(ip)


@pytest.mark.gpu
def test_native_bf16_upload_and_module_loading(backend, oracle, tmp_path):
    from kandle_b200.model_utils import Qwen3Config, Qwen3ForCausalLM
    from kandle_b200.core import Tensor
    dims = dict(vocab=96, hidden=64, inter=96, layers=2, heads=2, kv_heads=1, head_dim=64)
    w = synth.qwen3_weights(std=0.1, norm_jitter=0.05, **dims)
    bits = {k: (lib.f32_to_bf16_bits(v), "BF16") for k, v in w.items()}
    p = str(tmp_path / "qwen.safetensors")
    kio.save_file(bits, p)
    g = kio.loadSafetensor(p)
    lay = g.getLayer("model.embed_tokens.weight")
    t = kio.tensorFromSafetensorLayer(lay)                      # stays bf16 on the device
    assert t.dtype == "bfloat16" and t.shape == (96, 64)
    assert np.array_equal(t.dataAsync(), lay.to_float32())
    t32 = kio.tensorFromSafetensorLayer(lay, "float32")         # the reference's behaviour on request
    assert t32.dtype == "float32" and np.array_equal(t32.dataAsync(), lay.to_float32())
    cfg = Qwen3Config(vocabSize=96, hiddenSize=64, intermediateSize=96, numHiddenLayers=2, numAttentionHeads=2,
                      numKeyValueHeads=1, headDim=64)
    model = Qwen3ForCausalLM(cfg)
    res = kio.loadModuleFromSafetensor(model, g, keyMapper=lambda k: None if k == "lm_head.weight" else k, strict=False)
    assert set(res["missingKeys"]) <= {"lm_head.weight"} and not res["unexpectedKeys"]
    ids = synth.token_ids("st.ids", (2, 9), 96)
    wr = {k: lib.round_to_bf16(v) for k, v in w.items()}
    ocfg = oracle.Qwen3Config(vocab_size=96, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=2,
                              num_key_value_heads=1, head_dim=64)
    ref = oracle.Qwen3Oracle(ocfg, wr).logits(ids)
    got = model.forward(Tensor(ids)).dataAsync()
    assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()
    with pytest.raises(KeyError):
        kio.loadModuleFromSafetensor(model, g, keyMapper=lambda k: k + ".nope")
    # the fused engine straight from the checkpoint
    from kandle_b200.engine import Qwen3Engine
    ecfg = Qwen3Config(vocabSize=96, hiddenSize=64, intermediateSize=96, numHiddenLayers=2, numAttentionHeads=2,
                       numKeyValueHeads=1, headDim=64, dtype="bfloat16")
    eng = Qwen3Engine(ecfg, kio.SafetensorStateDict(g), 2, 32)
    _, logits = eng.prefill(ids, all_logits=True)
    assert np.abs(logits.dataAsync() - ref).max() <= 3e-2 * max(1.0, np.abs(ref).max())
    eng.dispose()
