"""Headline benchmark: Qwen3-0.6B-architecture bf16 prefill + greedy decode, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (`config.workload` = "qwen3-0.6b-bf16-b32-p2048-d256"): random-init weights N(0, 0.02) of
the Qwen3-0.6B architecture (28 layers, hidden 1024, 16 q / 8 kv heads x 128, MLP 3072, vocab
151936, tied lm_head), 32 independent sequences of 2048 uniform-random prompt tokens, then 256
greedy decode steps against a KV cache.  One "step" of the benchmark is that whole job: 32 x 2048
prompt tokens prefilled + 32 x 256 tokens generated = 73 728 tokens.  With N GPUs every rank runs
its own 32 sequences (independent units, no data-path collective): weak scaling.

  value   tokens/s with the prompt ids already resident in HBM, timed with CUDA events on the
          library's stream, max over ranks.
  e2e     the same job through the public host API (`Qwen3Engine.generate`): prompt ids start in
          pinned host memory and are copied in every step; every decode step's token ids are read
          back to the host (as the reference's generation loop does).
  roofline  the dominant kernel by time (split-KV decode attention, HBM-bound) timed alone with CUDA
          events at the mean context length; prefill GEMM / attention figures ride along in
          `roofline_other`.
  cpu_baseline  the CPU oracle (fp32 restatement of the reference's arithmetic, OpenMP) on a bounded
          sample of the same workload on this box's host cores (rank 0, N=1 only).

`--impl reference` times only that CPU arm (the reference has no runnable CPU or GPU path on this
box: it is WebGPU-only TypeScript and its JS CPU backend is not in its repository).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ARCH = dict(vocab=151936, hidden=1024, inter=3072, layers=28, heads=16, kv_heads=8, head_dim=128)
ARCH_4B = dict(vocab=151936, hidden=2560, inter=9728, layers=36, heads=32, kv_heads=8, head_dim=128)
METRIC = "qwen3_0.6b_bf16_prefill_decode_tokens_per_s"
METRIC_4B = "qwen3_4b_bf16_tensor_parallel_prefill_decode_tokens_per_s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen3-0.6b", choices=["qwen3-0.6b", "qwen3-4b-tp"],
                    help="qwen3-0.6b: 32 sequences per GPU, replicated model (default, the headline); "
                         "qwen3-4b-tp: 8 x 4096 + 128 steps, one model tensor-parallel over all ranks (strong scaling)")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prompt", type=int, default=None)
    ap.add_argument("--decode", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--vocab", type=int, default=ARCH["vocab"])
    ap.add_argument("--cpu-sample", default="1x256+8", help="cpu baseline sample: <seqs>x<prompt>+<decode steps>")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    a = ap.parse_args()
    tp = a.workload == "qwen3-4b-tp"
    a.arch = dict(ARCH_4B if tp else ARCH)
    a.batch = a.batch or (8 if tp else 32)
    a.prompt = a.prompt or (4096 if tp else 2048)
    a.decode = a.decode or (128 if tp else 256)
    a.layers = a.layers or a.arch["layers"]
    a.metric = METRIC_4B if tp else METRIC
    a.tp = tp
    return a


def workload_name(a) -> str:
    base = "qwen3-4b-tp" if a.tp else "qwen3-0.6b"
    full = a.layers == a.arch["layers"] and a.vocab == 151936
    return f"{base}-bf16-b{a.batch}-p{a.prompt}-d{a.decode}" + ("" if full else f"-L{a.layers}-V{a.vocab}")


# --------------------------------------------------------------------------- clocks sampler
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.thread, self.gpu = [], None, None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.time(), line.strip()))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()   # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], None, [], set()
        for ts, line in self.rows:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not (t0 <= ts <= t1 + 0.3):
                continue
            try:
                sm.append(float(f[1])); mx = float(f[2]); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arm (oracle)
def cpu_arm(sample: str, layers: int, vocab: int, arch: dict = ARCH):
    """Times the CPU oracle on `<seqs>x<prompt>+<steps>`: prefill + greedy decode with a KV cache,
    fp32, all host threads.  Returns (tokens/s, description, threads)."""
    from kandle_b200 import lib, synth
    from oracle import oracle as orc
    orc.build()
    seqs, rest = sample.split("x")
    prompt, steps = rest.split("+")
    seqs, prompt, steps = int(seqs), int(prompt), int(steps)
    dims = dict(arch, layers=layers, vocab=vocab)
    w = synth.qwen3_weights(**dims)
    w = {k: lib.round_to_bf16(v) for k, v in w.items()}
    cfg = orc.Qwen3Config(vocab_size=vocab, hidden_size=dims["hidden"], intermediate_size=dims["inter"],
                          num_hidden_layers=layers, num_attention_heads=dims["heads"], num_key_value_heads=dims["kv_heads"],
                          head_dim=dims["head_dim"])
    model = orc.Qwen3Oracle(cfg, w)
    ids = synth.token_ids("bench.cpu.ids", (seqs, prompt), vocab)
    t0 = time.perf_counter()
    model.greedy_generate(ids, steps, max_seq_len=prompt + steps)
    dt = time.perf_counter() - t0
    tokens = seqs * (prompt + steps)
    desc = f"{seqs} sequence(s) x {prompt} prompt tokens + {steps} greedy decode steps, fp32, {layers} layers, vocab {vocab}"
    return tokens / dt, desc, orc.num_threads(), dt


def run_reference(a) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    desc, threads = "", 1
    for i in range(a.warmup + a.steps):
        v, desc, threads, dt = cpu_arm(a.cpu_sample, a.layers, a.vocab, a.arch)
        if i >= a.warmup:
            vals.append((v, dt))
        if i == 0 and dt > 60:     # keep the whole run within minutes
            vals = vals or [(v, dt)]
            break
    v = float(np.mean([x[0] for x in vals]))
    ms = float(np.mean([x[1] for x in vals])) * 1e3
    line = {
        "impl": "reference", "metric": a.metric, "value": v, "unit": "tokens/s", "n_gpus": a.gpus, "steps": len(vals),
        "warmup": a.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if a.tp else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(a), "note": "CPU arm runs a bounded sample of the workload: " + desc},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "reference_note": "the reference (final-kk/kandle) has no runnable path here: WebGPU-only TypeScript, no JS runtime, "
                          "its JS CPU backend is not in its repository; this arm times the CPU restatement of its arithmetic",
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- our arm
def run_ours(a) -> None:
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import kandle_b200
    from kandle_b200 import core, lib, synth
    from kandle_b200.backend import CudaEvent
    from kandle_b200.core import Tensor
    from kandle_b200.engine import Qwen3Engine
    from kandle_b200.model_utils import Qwen3Config

    be = kandle_b200.init(local_rank)
    dims = dict(a.arch, layers=a.layers, vocab=a.vocab)
    tp_size = world if a.tp else 1
    if tp_size > 1:
        from kandle_b200 import parallel
        def bcast(obj):
            box = [obj]
            dist.broadcast_object_list(box, src=0)
            return box[0]
        parallel.init_tensor_parallel(rank, world, bcast)
    # one tensor at a time; replicated model (every rank identical) or this rank's tensor-parallel slice
    weights = synth.LazyQwen3Weights(**dims, shard=(rank, world) if tp_size > 1 else None)
    cfg = Qwen3Config(vocabSize=a.vocab, hiddenSize=dims["hidden"], intermediateSize=dims["inter"], numHiddenLayers=a.layers,
                      numAttentionHeads=dims["heads"], numKeyValueHeads=dims["kv_heads"], headDim=dims["head_dim"], dtype="bfloat16")
    B, S, T = a.batch, a.prompt, a.decode
    max_s = S + T + 16
    eng = Qwen3Engine(cfg, weights, B, max_s, tp_size=tp_size)
    del weights
    # data parallel: each rank its own sequences; tensor parallel: every rank the same batch
    ids_host = synth.token_ids("bench.ids.tp" if a.tp else f"bench.ids.rank{rank}", (B, S), a.vocab)
    ids_dev = Tensor(ids_host)                                            # resident copy for `value`
    pinned = ctypes.c_void_p()
    lib.call("kd_host_alloc_pinned", ctypes.c_uint64(ids_host.nbytes), ctypes.byref(pinned))
    ctypes.memmove(pinned, ids_host.ctypes.data, ids_host.nbytes)
    tok_pinned = ctypes.c_void_p()
    lib.call("kd_host_alloc_pinned", ctypes.c_uint64(B * 8), ctypes.byref(tok_pinned))
    ids_stage = core.empty((B, S), "int32")

    def sync_all():
        be.synchronize()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    def job_device():
        """prefill + T greedy tokens, ids resident on the device, no host read-back"""
        tok = eng.prefill(ids_dev)
        if T > 1:
            eng.start_decode(tok, use_graph=True)
            for _ in range(1, T):
                eng.decode_step()

    def job_e2e():
        """the same job through host buffers: H2D of the prompt, D2H of every step's tokens"""
        lib.call("kd_upload_async", ctypes.c_uint64(ids_stage._handle.storage.handle), ctypes.c_uint64(0), pinned,
                 ctypes.c_uint64(ids_host.nbytes))
        tok = eng.prefill(ids_stage)
        out = np.empty((B, T), dtype=np.int64)
        host = np.ctypeslib.as_array(ctypes.cast(tok_pinned, ctypes.POINTER(ctypes.c_int64)), shape=(B,))
        def read(t, i):
            lib.call("kd_download_async", ctypes.c_uint64(t._handle.storage.handle), ctypes.c_uint64(0), tok_pinned, ctypes.c_uint64(B * 8))
            be.synchronize()
            out[:, i] = host
        read(tok, 0)
        if T > 1:
            eng.start_decode(tok, use_graph=True)
            for i in range(1, T):
                read(eng.decode_step(), i)
        return out

    # ---- warm-up (also captures the decode graph and sizes scratch)
    for _ in range(max(a.warmup, 1)):
        job_device()
    job_e2e()
    sync_all()

    sampler = ClockSampler(local_rank)
    sampler.start()
    t_wall0 = time.time()
    # ---- timed: device-resident
    be.launch_count(reset=True)
    e0, e1 = CudaEvent(), CudaEvent()
    sync_all()
    e0.record()
    for _ in range(a.steps):
        job_device()
    e1.record()
    sync_all()
    ms_dev = e0.elapsed_ms(e1) / a.steps
    launches = be.launch_count() // a.steps
    # prefill / decode split (one extra job, timed in two parts)
    p0, p1, p2 = CudaEvent(), CudaEvent(), CudaEvent()
    p0.record()
    tok = eng.prefill(ids_dev)
    p1.record()
    if T > 1:
        eng.start_decode(tok, use_graph=True)
        for _ in range(1, T):
            eng.decode_step()
    p2.record()
    be.synchronize()
    ms_prefill, ms_decode = p0.elapsed_ms(p1), p1.elapsed_ms(p2)
    # ---- timed: end to end through host buffers
    sync_all()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        job_e2e()
    sync_all()
    ms_e2e = (time.perf_counter() - t0) * 1e3 / a.steps
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1)

    # ---- dominant kernel alone: split-KV decode attention at the mean decode context
    ctx_mean = S + T // 2
    d = eng._decode
    roofline, other = None, {}
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak, hbm_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
    tc_peak, tc_src = (peaks["bf16_tflops"], "measured") if "bf16_tflops" in peaks else (1590.0, "fallback")
    if d is not None and T > 1:
        q_bh1d = d["q"].permute([0, 2, 1, 3])
        o_bh1d = d["attn"].permute([0, 2, 1, 3])
        n_l = len(eng.layers)
        def attn_all_layers():
            for li in range(n_l):   # one launch per layer, each on its own (cold) cache slab
                lib.call("kd_attention_decode", ctypes.byref(q_bh1d._handle.c()), ctypes.byref(eng.k_cache[li]._handle.c()),
                         ctypes.byref(eng.v_cache[li]._handle.c()), None, ctx_mean, ctypes.c_float(eng.scale), 0,
                         ctypes.byref(o_bh1d._handle.c()))
        attn_all_layers()
        k0, k1 = CudaEvent(), CudaEvent()
        k0.record()
        reps = 5
        for _ in range(reps):
            attn_all_layers()
        k1.record()
        us = k0.elapsed_ms(k1) * 1e3 / (reps * n_l)
        alg_bytes = 2.0 * B * (dims["kv_heads"] // tp_size) * ctx_mean * dims["head_dim"] * 2
        ach = alg_bytes / (us * 1e-6) / 1e9
        roofline = {"kernel": "flash_attention_tcgen05_kernel<decode> (+ decode_combine_kernel when the keys are split)", "bound": "hbm", "achieved": ach,
                    "peak": hbm_peak, "peak_source": hbm_src, "unit": "GB/s", "frac": ach / hbm_peak,
                    # dram__bytes_read+write of one ncu capture at B=32, Hkv=8, ctx=2176 (289.4 MB for 285.2 MB
                    # algorithmic); traffic is proportional to the keys read, so other shapes are scaled
                    "traffic": alg_bytes * (289.37e6 / 285.212672e6),
                    "algorithmic_bytes_per_launch": alg_bytes, "us_per_launch": us, "context": ctx_mean}
        if d.get("chain") and n_l > 1:
            # the per-layer chain kernel (o_proj .. next QKV), one launch per layer so that weights stream from HBM
            attn2d = d["attn"].view(B, eng.Hq * eng.D)
            eps = ctypes.c_float(eng.cfg.rmsNormEps)
            r_ = lambda t: ctypes.byref(t._handle.c())  # noqa: E731
            def chain_all_layers():
                for li in range(n_l - 1):
                    lw_ = eng.layers[li]
                    lib.call("kd_decode_layer_chain", r_(attn2d), r_(lw_["wo"]), r_(d["h"]), r_(lw_["post_norm"]), r_(lw_["wgu"]),
                             r_(lw_["wdown"]), r_(eng.layers[li + 1]["in_norm"]), eps, r_(eng.layers[li + 1]["wqkv"]), r_(d["h1"]),
                             r_(d["h"]), r_(d["x"]), r_(d["act"]), r_(d["qkv_p"]))
            chain_all_layers()
            c0, c1 = CudaEvent(), CudaEvent()
            c0.record()
            for _ in range(reps):
                chain_all_layers()
            c1.record()
            us_c = c0.elapsed_ms(c1) * 1e3 / (reps * (n_l - 1))
            wbytes = 2.0 * (eng.H * eng.Hq * eng.D + 3 * eng.I * eng.H + eng.nqkv * eng.H)
            other["decode_chain"] = {"bound": "hbm", "achieved": wbytes / (us_c * 1e-6) / 1e9, "peak": hbm_peak, "peak_source": hbm_src,
                                     "unit": "GB/s", "frac": wbytes / (us_c * 1e-6) / 1e9 / hbm_peak, "us_per_launch": us_c,
                                     "note": "latency-bound: six dependent phases per launch; eager launches, gaps included"}
    # prefill GEMM + attention, timed alone on the prefill buffers
    w = eng._bufs(B, S)
    lw = eng.layers[0]
    def timed(fn, reps=3):
        fn()
        a0, a1 = CudaEvent(), CudaEvent()
        a0.record()
        for _ in range(reps):
            fn()
        a1.record()
        return a0.elapsed_ms(a1) / reps
    Tt = B * S
    ms = timed(lambda: eng._linear(w["x"], lw["wgu"], w["act"], epi=2))
    fl = 2.0 * Tt * 2 * (dims["inter"] // tp_size) * dims["hidden"]
    other["gemm_gate_up_swiglu"] = {"bound": "tensor", "achieved": fl / ms / 1e9, "peak": tc_peak, "peak_source": tc_src,
                                    "unit": "TFLOP/s", "frac": fl / ms / 1e9 / tc_peak, "us_per_launch": ms * 1e3}
    ms = timed(lambda: eng._linear(w["x"], lw["wqkv"], w["qkv"]))
    fl = 2.0 * Tt * eng.nqkv * dims["hidden"]
    other["gemm_qkv"] = {"bound": "tensor", "achieved": fl / ms / 1e9, "peak": tc_peak, "peak_source": tc_src, "unit": "TFLOP/s",
                         "frac": fl / ms / 1e9 / tc_peak, "us_per_launch": ms * 1e3}
    q_bhsd, o_bhsd = w["q"].permute([0, 2, 1, 3]), w["attn"].permute([0, 2, 1, 3])
    kp, vp = eng.k_cache[0].slice(f":{B}, :, :{S}, :"), eng.v_cache[0].slice(f":{B}, :, :{S}, :")
    ms = timed(lambda: lib.call("kd_flash_attention", ctypes.byref(q_bhsd._handle.c()), ctypes.byref(kp._handle.c()),
                                ctypes.byref(vp._handle.c()), ctypes.byref(o_bhsd._handle.c()), ctypes.c_float(eng.scale), 1))
    fl = 4.0 * B * (dims["heads"] // tp_size) * dims["head_dim"] * (S * (S + 1) / 2)
    other["flash_attention_prefill"] = {"bound": "tensor", "achieved": fl / ms / 1e9, "peak": tc_peak, "peak_source": tc_src,
                                        "unit": "TFLOP/s", "frac": fl / ms / 1e9 / tc_peak, "us_per_launch": ms * 1e3}
    be.synchronize()

    # ---- max over ranks
    if dist is not None:
        import torch
        t = torch.tensor([ms_dev, ms_e2e, ms_prefill, ms_decode], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_dev, ms_e2e, ms_prefill, ms_decode = [float(x) for x in t.tolist()]
    tokens_rank = B * (S + T)
    tokens_all = tokens_rank * (1 if a.tp else world)     # tensor parallel: all ranks work on the same tokens

    cpu = None
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        v, desc, threads, _ = cpu_arm(a.cpu_sample, a.layers, a.vocab, a.arch)
        cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc}

    if rank == 0:
        per_layer_params = dims["hidden"] * ((dims["heads"] + 2 * dims["kv_heads"]) * dims["head_dim"]) + \
            dims["hidden"] * dims["heads"] * dims["head_dim"] + 3 * dims["hidden"] * dims["inter"]
        flops_prefill = B * S * (2.0 * per_layer_params * a.layers) + 4.0 * B * dims["heads"] * dims["head_dim"] * (S * (S + 1) / 2) * a.layers
        line = {
            "metric": a.metric, "value": tokens_all / (ms_dev * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "strong" if a.tp else "weak",
            "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(a), "sequences_per_gpu": B, "prompt_tokens": S, "decode_steps": T,
                       "tokens_per_step_per_gpu": tokens_rank, "logits": "last position only (select before the tied lm_head)",
                       "l2": "inputs larger than L2 (bf16 weights and KV cache, GBs per pass)", "parallelism": f"tp{world}" if a.tp else f"dp{world}"},
            "e2e": {"value": tokens_all / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(ids_host.nbytes),
                    "d2h_bytes_per_step": int(B * 8 * T), "ms_per_step": ms_e2e},
            "gpu_launches": int(launches),
            "phases": {"prefill_ms": ms_prefill, "decode_ms": ms_decode,
                       "prefill_tokens_per_s": B * S * (tokens_all // tokens_rank) / (ms_prefill * 1e-3),
                       "decode_tokens_per_s": B * max(T - 1, 1) * (tokens_all // tokens_rank) / (max(ms_decode, 1e-9) * 1e-3),
                       "prefill_tflops_per_gpu": flops_prefill / (tp_size if a.tp else 1) / (ms_prefill * 1e-3) / 1e12,
                       "prefill_frac_of_tensor_peak": flops_prefill / (tp_size if a.tp else 1) / (ms_prefill * 1e-3) / 1e12 / tc_peak},
            "roofline": roofline, "roofline_other": other, "cpu_baseline": cpu, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    eng.dispose()                 # graphs that captured NCCL work must go before the communicator
    if tp_size > 1:
        lib.call("kd_comm_destroy")
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
