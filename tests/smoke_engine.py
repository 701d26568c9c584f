"""Small end-to-end check used by the smoke entry point: a tiny Qwen3 through the eager operator
path (and the fused engine when available) against an oracle object passed in by the caller."""
from __future__ import annotations

import numpy as np

from kandle_b200 import synth
from kandle_b200.core import Tensor
from kandle_b200.model_utils import Qwen3Config, Qwen3ForCausalLM


def run(backend, orc) -> None:
    dims = dict(vocab=211, hidden=128, inter=192, layers=2, heads=4, kv_heads=2, head_dim=64)
    w = synth.qwen3_weights(std=0.08, **dims)
    cfg = Qwen3Config(vocabSize=211, hiddenSize=128, intermediateSize=192, numHiddenLayers=2, numAttentionHeads=4,
                      numKeyValueHeads=2, headDim=64)
    model = Qwen3ForCausalLM(cfg)
    model.loadStateDict(w)
    ocfg = orc.Qwen3Config(vocab_size=211, hidden_size=128, intermediate_size=192, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=64)
    oracle_model = orc.Qwen3Oracle(ocfg, w)
    ids = synth.token_ids("smoke.ids", (2, 12), 211)
    got = model.forward(Tensor(ids)).dataAsync()
    ref = oracle_model.logits(ids)
    err = float(np.abs(got - ref).max() / np.abs(ref).max())
    assert err <= 1e-4, f"tiny Qwen3 prefill differs from the oracle: {err}"
    toks = model.generateGreedy(Tensor(ids), 4)
    assert np.array_equal(toks, oracle_model.greedy_generate(ids, 4).astype(np.int64)), "greedy tokens differ"
    print(f"smoke: tiny Qwen3 fp32 prefill error {err:.2e}, 4 greedy steps identical to the oracle")

    # fused bf16 engine (tensor-core GEMMs, tcgen05 attention, split-KV decode, graph replay)
    from kandle_b200 import lib
    from kandle_b200.engine import Qwen3Engine
    dims = dict(vocab=512, hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=128)
    wb = {k: lib.round_to_bf16(v) for k, v in synth.qwen3_weights(std=0.04, **dims).items()}
    cfg = Qwen3Config(vocabSize=512, hiddenSize=256, intermediateSize=512, numHiddenLayers=2, numAttentionHeads=4,
                      numKeyValueHeads=2, headDim=128, dtype="bfloat16")
    eng = Qwen3Engine(cfg, wb, 2, 192)
    ocfg = orc.Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    om = orc.Qwen3Oracle(ocfg, wb)
    ids = synth.token_ids("smoke.ids2", (2, 140), 512)
    tok, logits = eng.prefill(ids, all_logits=True)
    ref = om.logits(ids)
    e = np.abs(logits.dataAsync() - ref)
    assert np.quantile(e, 0.999) <= 2e-2 and e.max() <= 3e-2, f"bf16 engine logits differ from the oracle: max {e.max():.3e}"
    toks = eng.generate(ids, 4)
    assert (toks == om.greedy_generate(ids, 4).astype(np.int64)).mean() >= 0.75, "bf16 engine greedy tokens differ"
    eng.dispose()
    print(f"smoke: bf16 engine logits max-abs error {e.max():.2e} (p99.9 {np.quantile(e, 0.999):.2e}); prefill + graph decode ok")
