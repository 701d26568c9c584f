"""CPU tests of the multi-GPU host logic: sequence sharding, tensor-parallel weight slicing (the sum
of the per-rank partial products equals the unsharded product), and a world-size-2 gloo run in which
each rank plays one GPU with the CPU oracle as its compute."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_covers_everything_once():
    from kandle_b200.parallel import shard_range
    for n in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_tensor_parallel_slices_sum_to_the_full_layer(oracle):
    from kandle_b200 import synth
    from kandle_b200.parallel import shard_qwen3_weights
    dims = dict(vocab=64, hidden=64, inter=96, layers=1, heads=4, kv_heads=2, head_dim=32)
    w = synth.qwen3_weights(std=0.1, **dims)
    x = synth.normal("x", (5, 128))          # attention output [tokens, Hq*D]
    a = synth.normal("a", (5, 96))           # MLP activation [tokens, I]
    full_o = oracle.linear(x, w["model.layers.0.self_attn.o_proj.weight"])
    full_d = oracle.linear(a, w["model.layers.0.mlp.down_proj.weight"])
    for world in (1, 2):
        po, pd, q_rows = 0, 0, []
        for r in range(world):
            s = shard_qwen3_weights(w, heads=4, kv_heads=2, head_dim=32, rank=r, world=world)
            hq = 4 // world
            po = po + oracle.linear(x[:, r * hq * 32:(r + 1) * hq * 32], s["model.layers.0.self_attn.o_proj.weight"])
            pd = pd + oracle.linear(a[:, r * 96 // world:(r + 1) * 96 // world], s["model.layers.0.mlp.down_proj.weight"])
            q_rows.append(s["model.layers.0.self_attn.q_proj.weight"])
            assert s["model.embed_tokens.weight"].shape == (64, 64)
        assert np.abs(po - full_o).max() < 1e-5 and np.abs(pd - full_d).max() < 1e-5
        assert np.array_equal(np.concatenate(q_rows), w["model.layers.0.self_attn.q_proj.weight"])
    with pytest.raises(ValueError):
        shard_qwen3_weights(w, heads=4, kv_heads=2, head_dim=32, rank=0, world=3)


WORKER = r'''
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["KD_ROOT"])
from kandle_b200 import synth
from kandle_b200.parallel import shard_range, shard_qwen3_weights
from oracle import oracle as orc
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
dims = dict(vocab=97, hidden=64, inter=96, layers=2, heads=4, kv_heads=2, head_dim=32)
w = synth.qwen3_weights(std=0.1, **dims)
cfg = orc.Qwen3Config(vocab_size=97, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32)
ids = synth.token_ids("ids", (5, 9), 97)
# (1) independent sequences sharded over ranks: gathered result equals the single-rank result
b, e = shard_range(5, rank, world)
mine = orc.Qwen3Oracle(cfg, w).greedy_generate(ids[b:e], 3) if e > b else np.zeros((0, 3), np.int32)
parts = [None] * world
dist.all_gather_object(parts, mine)
# (2) tensor parallel: partial o_proj products all-reduced over ranks equal the full product
s = shard_qwen3_weights(w, heads=4, kv_heads=2, head_dim=32, rank=rank, world=world)
x = synth.normal("x", (6, 128))
hq = 4 // world
part = torch.tensor(orc.linear(x[:, rank * hq * 32:(rank + 1) * hq * 32], s["model.layers.1.self_attn.o_proj.weight"]))
dist.all_reduce(part)
# (3) max-over-ranks of a timing, as the benchmark reports it
t = torch.tensor([10.0 + rank], dtype=torch.float64)
dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0:
    full = orc.Qwen3Oracle(cfg, w).greedy_generate(ids, 3)
    assert np.array_equal(np.concatenate(parts), full)
    assert np.abs(part.numpy() - orc.linear(x, w["model.layers.1.self_attn.o_proj.weight"])).max() < 1e-5
    assert t.item() == 10.0 + world - 1
    print("gloo-ok")
dist.barrier()
dist.destroy_process_group()
'''


def test_world_size_2_gloo_ranks(tmp_path, oracle):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, KD_ROOT=ROOT, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29517", str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "gloo-ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
