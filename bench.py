"""Headline benchmark: Qwen3-0.6B-architecture bf16 prefill + greedy decode, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

Headline workload (`config.workload` = "qwen3-0.6b-bf16-b32-p2048-d256"): random-init weights
N(0, 0.02) of the Qwen3-0.6B architecture (28 layers, hidden 1024, 16 q / 8 kv heads x 128, MLP 3072,
vocab 151936, tied lm_head), 32 independent sequences of 2048 uniform-random prompt tokens, then 256
greedy decode steps against a KV cache.  One "step" of the benchmark is that whole job: 32 x 2048
prompt tokens prefilled + 32 x 256 tokens generated = 73 728 tokens.  With N GPUs the 32 sequences
are sharded, 32/N per rank, weights replicated, no data-path collective: STRONG scaling.

  value   tokens/s of the whole job with the prompt ids already resident in HBM, timed with CUDA
          events on the library's stream, max over ranks.
  e2e     the same job through the public host API: each rank's prompt ids start in pinned host
          memory and are copied in every step; every decode step's token ids are read back to the
          host (as the reference's generation loop does).
  parity_ok  N > 1: the tokens the N ranks generated, gathered on rank 0, equal bit for bit the
          tokens rank 0 generates alone for all 32 sequences in micro-batches of 32/N.  N = 1: the
          timed run's tokens equal an eager re-run of the same job (no graph replay).
  roofline  the dominant kernel by time (split-KV decode attention, HBM-bound) timed alone with CUDA
          events at the mean context length; GEMM / attention / lm_head / chain figures ride along in
          `roofline_other`, each against the measured and the nominal ceiling.
  cpu_baseline  the CPU oracle (fp32 restatement of the reference's arithmetic, OpenMP) on a bounded
          sample of the same workload on this box's host cores (rank 0, N=1 only).
  extras  further records in the same line, each a small timed run of its own:
          `weak_dp`     (N > 1) 32 sequences on EVERY rank, the weak-scaling figure;
          `tp_4b`       Qwen3-4B shapes, 8 x 4096 prompt + 128 decode steps, ONE model tensor-parallel
                        over the N ranks (N = 1: the same model on one GPU), with the time of its
                        all-reduces measured alone;
          `whisper_c5`  Whisper-small encoder, 64 clips of 30 s sharded over the N ranks.

`--impl reference` times only the CPU arm (the reference has no runnable CPU or GPU path on this
box: it is WebGPU-only TypeScript and its JS CPU backend is not in its repository).
"""
from __future__ import annotations

import argparse
import ctypes
import hashlib
import importlib.util
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
NOMINAL_HBM_GBS = 8000.0        # vendor figure for HBM3e on B200
NOMINAL_BF16_TFLOPS = 2250.0    # vendor dense bf16 figure
TOTAL_SEQUENCES = 32


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sequences", type=int, default=TOTAL_SEQUENCES, help="sequences in the whole job (sharded over the ranks)")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--decode", type=int, default=256)
    ap.add_argument("--layers", type=int, default=ARCH["layers"])
    ap.add_argument("--vocab", type=int, default=ARCH["vocab"])
    ap.add_argument("--cpu-sample", default="4x512+16", help="cpu baseline sample: <seqs>x<prompt>+<decode steps>")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline only (no weak_dp / tp_4b / whisper_c5 records)")
    ap.add_argument("--extras", default="weak_dp,tp_4b,whisper_c5")
    ap.add_argument("--tp-layers", type=int, default=ARCH_4B["layers"])
    return ap.parse_args()


def workload_name(a) -> str:
    full = a.layers == ARCH["layers"] and a.vocab == ARCH["vocab"]
    return f"qwen3-0.6b-bf16-b{a.sequences}-p{a.prompt}-d{a.decode}" + ("" if full else f"-L{a.layers}-V{a.vocab}")


def load_peaks():
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    hbm = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
    tc = (peaks["bf16_tflops"], "measured") if "bf16_tflops" in peaks else (1590.0, "fallback")
    return hbm, tc


def roof(bound: str, achieved: float, peaks, **more) -> dict:
    (hbm, hbm_src), (tc, tc_src) = peaks
    peak, src, nominal, unit = (hbm, hbm_src, NOMINAL_HBM_GBS, "GB/s") if bound == "hbm" else (tc, tc_src, NOMINAL_BF16_TFLOPS, "TFLOP/s")
    d = {"bound": bound, "achieved": achieved, "peak": peak, "peak_source": src, "unit": unit, "frac": achieved / peak,
         "peak_nominal": nominal, "frac_nominal": achieved / nominal}
    d.update(more)
    return d


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
def _round_to_bf16(a: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16 (ties to even) -> float32, in numpy: the CPU arm loads no CUDA library."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = (u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) & np.uint32(0xFFFF0000)
    return r.view(np.float32).reshape(a.shape)


def _synth_module():
    """kandle_b200/synth.py loaded by path (numpy only), without importing the package and its library."""
    spec = importlib.util.spec_from_file_location("_bench_synth", os.path.join(ROOT, "kandle_b200", "synth.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


_CPU_MODEL = {}


def cpu_arm(sample: str, layers: int, vocab: int):
    """Times the CPU oracle on `<seqs>x<prompt>+<steps>`: prefill + greedy decode with a KV cache,
    fp32, all host threads.  Returns (tokens/s, description, threads, seconds)."""
    from oracle import oracle as orc
    orc.build()
    orc.set_num_threads(os.cpu_count() or 1)     # a launcher may have exported OMP_NUM_THREADS=1
    synth = _synth_module()
    seqs, rest = sample.split("x")
    prompt, steps = rest.split("+")
    seqs, prompt, steps = int(seqs), int(prompt), int(steps)
    dims = dict(ARCH, layers=layers, vocab=vocab)
    key = (layers, vocab)
    if key not in _CPU_MODEL:
        w = {k: _round_to_bf16(v) for k, v in synth.qwen3_weights(**dims).items()}
        cfg = orc.Qwen3Config(vocab_size=vocab, hidden_size=dims["hidden"], intermediate_size=dims["inter"],
                              num_hidden_layers=layers, num_attention_heads=dims["heads"], num_key_value_heads=dims["kv_heads"],
                              head_dim=dims["head_dim"])
        _CPU_MODEL.clear()
        _CPU_MODEL[key] = orc.Qwen3Oracle(cfg, w)
    model = _CPU_MODEL[key]
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
    t_begin = time.perf_counter()
    for i in range(a.warmup + a.steps):
        v, desc, threads, dt = cpu_arm(a.cpu_sample, a.layers, a.vocab)
        if i >= a.warmup:
            vals.append((v, dt))
        if time.perf_counter() - t_begin > 150:     # keep the whole run within minutes
            vals = vals or [(v, dt)]
            break
    v = float(np.mean([x[0] for x in vals]))
    ms = float(np.mean([x[1] for x in vals])) * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": a.gpus, "steps": len(vals),
        "warmup": a.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
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
class Bench:
    """State shared by the headline run and the extra records of one process (one rank)."""

    def __init__(self, a):
        self.a = a
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.dist = None
        self.torch = None
        if self.world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(self.local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist, self.torch = dist, torch
        import kandle_b200
        self.be = kandle_b200.init(self.local_rank)
        self.peaks = load_peaks()
        self.tp_ready = False

    # ---- plumbing
    def sync_all(self):
        self.be.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.dist is None:
            return [float(v) for v in values]
        t = self.torch.tensor(list(values), device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def timed_ms(self, fn, reps: int = 3, warm: int = 1) -> float:
        from kandle_b200.backend import CudaEvent
        for _ in range(warm):
            fn()
        e0, e1 = CudaEvent(), CudaEvent()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        return e0.elapsed_ms(e1) / reps

    def release_memory(self):
        import gc
        from kandle_b200 import lib
        gc.collect()
        lib.call("kd_empty_cache")

    def make_engine(self, dims: dict, layers: int, vocab: int, max_batch: int, max_s: int, tp_size: int = 1):
        from kandle_b200.engine import Qwen3Engine, RandomInit
        from kandle_b200.model_utils import Qwen3Config
        cfg = Qwen3Config(vocabSize=vocab, hiddenSize=dims["hidden"], intermediateSize=dims["inter"], numHiddenLayers=layers,
                          numAttentionHeads=dims["heads"], numKeyValueHeads=dims["kv_heads"], headDim=dims["head_dim"], dtype="bfloat16")
        # weights are drawn on the device (Philox4x32-10 `randn` kernel): identical on every rank, sliced per rank for TP
        return Qwen3Engine(cfg, RandomInit(seed=1234, std=0.02), max_batch, max_s, tp_size=tp_size, tp_rank=self.rank if tp_size > 1 else 0)

    # ---- jobs
    @staticmethod
    def job_device(eng, ids_dev, T: int):
        """prefill + T greedy tokens, ids resident on the device, no host read-back"""
        tok = eng.prefill(ids_dev)
        if T > 1:
            eng.start_decode(tok, use_graph=True)
            for _ in range(1, T):
                eng.decode_step()

    def job_e2e(self, eng, stage, pinned_ids, nbytes_ids, tok_pinned, B: int, T: int) -> np.ndarray:
        """the same job through host buffers: H2D of the prompt, D2H of every step's tokens"""
        from kandle_b200 import lib
        lib.call("kd_upload_async", ctypes.c_uint64(stage._handle.storage.handle), ctypes.c_uint64(0), pinned_ids, ctypes.c_uint64(nbytes_ids))
        tok = eng.prefill(stage)
        out = np.empty((B, T), dtype=np.int64)
        host = np.ctypeslib.as_array(ctypes.cast(tok_pinned, ctypes.POINTER(ctypes.c_int64)), shape=(B,))
        def read(t, i):
            lib.call("kd_download_async", ctypes.c_uint64(t._handle.storage.handle), ctypes.c_uint64(0), tok_pinned, ctypes.c_uint64(B * 8))
            self.be.synchronize()
            out[:, i] = host
        read(tok, 0)
        if T > 1:
            eng.start_decode(tok, use_graph=True)
            for i in range(1, T):
                read(eng.decode_step(), i)
        return out


def run_headline(bn: Bench) -> dict:
    """Config 3: `sequences` independent sequences sharded over the ranks."""
    a = bn.a
    from kandle_b200 import core, lib, parallel, synth
    from kandle_b200.backend import CudaEvent
    from kandle_b200.core import Tensor
    be, rank, world = bn.be, bn.rank, bn.world
    dims = dict(ARCH, layers=a.layers, vocab=a.vocab)
    S, T, N_SEQ = a.prompt, a.decode, a.sequences
    lo, hi = parallel.shard_range(N_SEQ, rank, world)
    B = hi - lo
    if B == 0:
        raise SystemExit(f"rank {rank}: no sequence to work on ({N_SEQ} sequences over {world} ranks)")
    max_s = S + T + 16
    # with several ranks every rank also runs the full batch once (weak_dp record) and rank 0 the reference micro-batches
    max_b = N_SEQ if world > 1 else B
    eng = bn.make_engine(dims, a.layers, a.vocab, max_b, max_s)
    bn.engine = eng
    ids_all = synth.token_ids("bench.ids", (N_SEQ, S), a.vocab)       # the same 32 prompts whatever the number of ranks
    ids_host = np.ascontiguousarray(ids_all[lo:hi])
    ids_dev = Tensor(ids_host)                                            # resident copy for `value`
    pinned = ctypes.c_void_p()
    lib.call("kd_host_alloc_pinned", ctypes.c_uint64(ids_host.nbytes), ctypes.byref(pinned))
    ctypes.memmove(pinned, ids_host.ctypes.data, ids_host.nbytes)
    tok_pinned = ctypes.c_void_p()
    lib.call("kd_host_alloc_pinned", ctypes.c_uint64(B * 8), ctypes.byref(tok_pinned))
    ids_stage = core.empty((B, S), "int32")

    # ---- warm-up (also captures the decode graph and sizes scratch)
    for _ in range(max(a.warmup, 1)):
        bn.job_device(eng, ids_dev, T)
    tokens_mine = bn.job_e2e(eng, ids_stage, pinned, ids_host.nbytes, tok_pinned, B, T)
    bn.sync_all()

    sampler = ClockSampler(bn.local_rank)
    sampler.start()
    t_wall0 = time.time()
    # ---- timed: device-resident
    be.launch_count(reset=True)
    e0, e1 = CudaEvent(), CudaEvent()
    bn.sync_all()
    e0.record()
    for _ in range(a.steps):
        bn.job_device(eng, ids_dev, T)
    e1.record()
    bn.sync_all()
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
    bn.sync_all()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        bn.job_e2e(eng, ids_stage, pinned, ids_host.nbytes, tok_pinned, B, T)
    bn.sync_all()
    ms_e2e = (time.perf_counter() - t0) * 1e3 / a.steps
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1)
    ms_dev, ms_e2e, ms_prefill, ms_decode = bn.max_over_ranks([ms_dev, ms_e2e, ms_prefill, ms_decode])

    # ---- kernels alone (rank 0's figures are reported); timed right after the jobs, before the long all-logits GEMMs
    # push the GPU deeper into its power cap
    roofline, other = kernel_rooflines(bn, eng, B, S, T, dims)

    # ---- the unmodified model code computes logits for every prompt position (for_causal_lm.ts:184-185):
    # time the extra work (final norm + tied lm_head over all B*S rows, fp32 logits) on top of the prefill,
    # one sequence at a time into a reused [S, V] buffer (all 65 536 x 151 936 fp32 logits would be 40 GB)
    ms_all_logits = None
    if rank == 0:
        w = eng._bufs(B, S)
        xa = core.empty((S, eng.H), "bfloat16")
        full = core.empty((S, eng.V), "float32")
        h3 = w["h"].view(B, S, eng.H)
        rows = [h3.select(0, b) for b in range(B)]
        def all_logits():
            for hb in rows:
                eng._norm(hb, eng.final_norm, xa)
                eng._linear(xa, eng.embed, full)
        ms_all_logits = bn.timed_ms(all_logits, reps=2)
        for t in rows + [h3, xa, full]:
            t.dispose()

    # ---- parity across ranks: the shards' tokens against rank 0's own run of all sequences in micro-batches of B
    parity = None
    if world > 1:
        torch, dist = bn.torch, bn.dist
        if N_SEQ % world == 0:
            mine = torch.tensor(tokens_mine, device="cuda")
            gathered = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine)
            if rank == 0:
                got = torch.cat(gathered, 0).cpu().numpy()
                want = np.concatenate([eng.generate(ids_all[i:i + B], T) for i in range(0, N_SEQ, B)], axis=0)
                full_batch = eng.generate(ids_all, T)
                parity = {"parity_ok": bool(np.array_equal(got, want)),
                          "tokens_sha256": hashlib.sha256(got.tobytes()).hexdigest()[:16],
                          "reference_run": f"rank 0 alone, {N_SEQ} sequences in micro-batches of {B}",
                          "same_as_one_batch_of_all_sequences": float((got == full_batch).mean()),
                          "note": "bitwise equality is asserted against the same per-call batch size: the split-KV factor of the "
                                  "decode attention follows the number of sequences per call, which changes the summation order"}
        else:
            parity = {"parity_ok": None, "note": f"{N_SEQ} sequences do not divide over {world} ranks evenly; not compared"}
        bn.sync_all()
    else:
        # one GPU: the tokens of the timed end-to-end run against the same job launched kernel by kernel
        # (no graph replay); parity against the CPU oracle is what tests/test_full_configs_gpu.py checks
        again = eng.generate(ids_all, T, use_graph=False)
        got = np.asarray(tokens_mine)
        parity = {"parity_ok": bool(np.array_equal(got, again)),
                  "tokens_sha256": hashlib.sha256(np.ascontiguousarray(got).tobytes()).hexdigest()[:16],
                  "reference_run": "the same sequences again with eager launches instead of the replayed decode graph"}

    tokens_all = N_SEQ * (S + T)
    per_layer_params = dims["hidden"] * ((dims["heads"] + 2 * dims["kv_heads"]) * dims["head_dim"]) + \
        dims["hidden"] * dims["heads"] * dims["head_dim"] + 3 * dims["hidden"] * dims["inter"]
    flops_prefill = B * S * (2.0 * per_layer_params * a.layers) + 4.0 * B * dims["heads"] * dims["head_dim"] * (S * (S + 1) / 2) * a.layers
    (hbm_peak, _), (tc_peak, _) = bn.peaks
    kv_bytes = 2.0 * a.layers * dims["kv_heads"] * dims["head_dim"] * 2 * (S + T / 2) * B
    w_bytes = 2.0 * (per_layer_params * a.layers + dims["vocab"] * dims["hidden"])
    decode_floor_ms = (kv_bytes + w_bytes) / (hbm_peak * 1e9) * 1e3
    line = {
        "metric": METRIC, "value": tokens_all / (ms_dev * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(a), "sequences_total": N_SEQ, "sequences_per_gpu": B, "prompt_tokens": S, "decode_steps": T,
                   "tokens_per_step": tokens_all, "logits": "last position only (select before the tied lm_head); see phases.prefill_all_logits_ms",
                   "weights": "random-init N(0, 0.02), drawn on the device by the randn kernel (Philox4x32-10, seed 1234)",
                   "l2": "inputs larger than L2 (bf16 weights and KV cache, GBs per pass)", "parallelism": f"dp{world}"},
        "e2e": {"value": tokens_all / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(ids_host.nbytes) * world,
                "d2h_bytes_per_step": int(B * 8 * T) * world, "ms_per_step": ms_e2e},
        "gpu_launches": int(launches),
        "phases": {"prefill_ms": ms_prefill, "decode_ms": ms_decode, "decode_ms_per_step": ms_decode / max(T - 1, 1),
                   "decode_hbm_floor_ms_per_step": decode_floor_ms, "decode_frac_of_hbm_floor": decode_floor_ms / (ms_decode / max(T - 1, 1)),
                   "prefill_tokens_per_s": N_SEQ * S / (ms_prefill * 1e-3),
                   "decode_tokens_per_s": N_SEQ * max(T - 1, 1) / (max(ms_decode, 1e-9) * 1e-3),
                   "prefill_tflops_per_gpu": flops_prefill / (ms_prefill * 1e-3) / 1e12,
                   "prefill_frac_of_tensor_peak": flops_prefill / (ms_prefill * 1e-3) / 1e12 / tc_peak,
                   "prefill_frac_of_nominal_tensor_peak": flops_prefill / (ms_prefill * 1e-3) / 1e12 / NOMINAL_BF16_TFLOPS,
                   "prefill_all_logits_ms": (ms_prefill + ms_all_logits) if ms_all_logits is not None else None,
                   "prefill_all_logits_note": "prefill plus final norm + tied lm_head over every prompt position (what the unmodified "
                                              "model code computes); rank 0's shard, logits written sequence by sequence into one reused fp32 buffer"},
        "roofline": roofline, "roofline_other": other, "clocks": clocks,
    }
    if parity is not None:
        line["parity"] = parity
        line["parity_ok"] = parity.get("parity_ok")
    for p in (pinned, tok_pinned):
        lib.call("kd_host_free_pinned", p)
    for t in (ids_dev, ids_stage):
        t.dispose()
    return line


def kernel_rooflines(bn: Bench, eng, B: int, S: int, T: int, dims: dict):
    from kandle_b200 import lib
    from kandle_b200.backend import CudaEvent
    d = eng._decode
    roofline, other = None, {}
    ctx_mean = S + T // 2
    r_ = lambda t: ctypes.byref(t._handle.c())  # noqa: E731
    if d is not None and T > 1:
        q_bh1d = d["q"].permute([0, 2, 1, 3])
        o_bh1d = d["attn"].permute([0, 2, 1, 3])
        n_l = len(eng.layers)
        caches = [(eng.k_cache[li].slice([slice(0, B), slice(None), slice(None), slice(None)]),
                   eng.v_cache[li].slice([slice(0, B), slice(None), slice(None), slice(None)])) for li in range(n_l)]
        def attn_all_layers():
            for kc, vc in caches:   # one launch per layer, each on its own (cold) cache slab
                lib.call("kd_attention_decode", r_(q_bh1d), r_(kc), r_(vc), None, ctx_mean, ctypes.c_float(eng.scale), 0, r_(o_bh1d))
        us = bn.timed_ms(attn_all_layers, reps=5) * 1e3 / n_l
        alg_bytes = 2.0 * B * dims["kv_heads"] * ctx_mean * dims["head_dim"] * 2
        roofline = roof("hbm", alg_bytes / (us * 1e-6) / 1e9, bn.peaks,
                        kernel="flash_attention_tcgen05_kernel<decode> (+ decode_combine_kernel when the keys are split)",
                        # scaled: dram__bytes_read+write of the ncu capture in profiles/flash_attention_decode_b32_ctx2176.md
                        # (289.37 MB for 285.21 MB algorithmic at B=32, Hkv=8, ctx=2176) times this launch's algorithmic bytes
                        traffic=alg_bytes * (289.37e6 / 285.212672e6), traffic_source="scaled from profiles/flash_attention_decode_b32_ctx2176.md",
                        algorithmic_bytes_per_launch=alg_bytes, us_per_launch=us, context=ctx_mean, sequences=B)
        wbytes = 2.0 * (eng.H * eng.Hq * eng.D + 3 * eng.I * eng.H + eng.nqkv * eng.H)
        attn2d = d["attn"].view(B, eng.Hq * eng.D)
        eps = ctypes.c_float(eng.cfg.rmsNormEps)
        if d.get("fused") and n_l > 1:
            def layer_all():
                for li in range(n_l - 1):
                    lw_, nl = eng.layers[li], eng.layers[li + 1]
                    lib.call("kd_decode_layer_fused", r_(attn2d), r_(lw_["wo"]), r_(d["h"]), r_(lw_["post_norm"]), r_(lw_["wgu"]),
                             r_(lw_["wdown"]), r_(nl["in_norm"]), eps, r_(nl["wqkv"]), r_(nl["q_norm"]), r_(nl["k_norm"]), r_(d["cos"]),
                             r_(d["sin"]), r_(d["pos"]), r_(caches[li + 1][0]), r_(caches[li + 1][1]), None, r_(d["q"]), r_(d["h"]), None)
            # the launches of all layers captured once and replayed: an eager loop of this kernel is bound
            # by the host (20 tensor arguments, 8 tensor maps and the launch plan per call) on a slow host
            layer_all()
            lib.call("kd_graph_begin")
            try:
                layer_all()
            finally:
                g_layers = ctypes.c_uint64(0)
                lib.call("kd_graph_end", ctypes.byref(g_layers))
            us_c = bn.timed_ms(lambda: lib.call("kd_graph_launch", g_layers), reps=5) * 1e3 / (n_l - 1)
            bn.be.synchronize()
            lib.call("kd_graph_destroy", g_layers)
            other["decode_layer_fused"] = roof("hbm", wbytes / (us_c * 1e-6) / 1e9, bn.peaks, us_per_launch=us_c, sequences=B,
                                               note="o_proj .. next layer's QKV + q/k-norm + RoPE + cache write in one launch; latency-bound "
                                                    "(four dependent phases); the launches of all layers replayed from a graph, gaps included")
        elif d.get("chain") and n_l > 1:
            def chain_all_layers():
                for li in range(n_l - 1):
                    lw_ = eng.layers[li]
                    lib.call("kd_decode_layer_chain", r_(attn2d), r_(lw_["wo"]), r_(d["h"]), r_(lw_["post_norm"]), r_(lw_["wgu"]),
                             r_(lw_["wdown"]), r_(eng.layers[li + 1]["in_norm"]), eps, r_(eng.layers[li + 1]["wqkv"]), r_(d["h1"]),
                             r_(d["h"]), r_(d["x"]), r_(d["act"]), r_(d["qkv_p"]))
            us_c = bn.timed_ms(chain_all_layers, reps=5) * 1e3 / (n_l - 1)
            other["decode_chain"] = roof("hbm", wbytes / (us_c * 1e-6) / 1e9, bn.peaks, us_per_launch=us_c, sequences=B,
                                         note="o_proj .. next QKV of one layer in one launch; latency-bound (dependent phases); eager launches, gaps included")
        # tied lm_head of the decode step: [B,H] x [V,H]^T, one pass over the embedding matrix
        us_l = bn.timed_ms(lambda: lib.call("kd_linear_bf16_skinny", r_(d["x"]), r_(eng.embed), 0, r_(d["logits"])), reps=10) * 1e3
        lbytes = 2.0 * eng.V * eng.H
        other["lm_head_skinny"] = roof("hbm", lbytes / (us_l * 1e-6) / 1e9, bn.peaks, us_per_launch=us_l, sequences=B,
                                       note="the embedding matrix (311 MB) exceeds L2, every launch streams it from HBM")
    # prefill GEMM + attention, timed alone on the prefill buffers
    w = eng._bufs(B, S)
    lw = eng.layers[0]
    Tt = B * S
    ms = bn.timed_ms(lambda: eng._linear(w["x"], lw["wgu"], w["act"], epi=2))
    fl = 2.0 * Tt * 2 * dims["inter"] * dims["hidden"]
    other["gemm_gate_up_swiglu"] = roof("tensor", fl / ms / 1e9, bn.peaks, us_per_launch=ms * 1e3, rows=Tt)
    ms = bn.timed_ms(lambda: eng._linear(w["x"], lw["wqkv"], w["qkv"]))
    fl = 2.0 * Tt * eng.nqkv * dims["hidden"]
    other["gemm_qkv"] = roof("tensor", fl / ms / 1e9, bn.peaks, us_per_launch=ms * 1e3, rows=Tt)
    q_bhsd, o_bhsd = w["q"].permute([0, 2, 1, 3]), w["attn"].permute([0, 2, 1, 3])
    kp, vp = eng.k_cache[0].slice(f":{B}, :, :{S}, :"), eng.v_cache[0].slice(f":{B}, :, :{S}, :")
    ms = bn.timed_ms(lambda: lib.call("kd_flash_attention", r_(q_bhsd), r_(kp), r_(vp), r_(o_bhsd), ctypes.c_float(eng.scale), 1))
    fl = 4.0 * B * dims["heads"] * dims["head_dim"] * (S * (S + 1) / 2)
    other["flash_attention_prefill"] = roof("tensor", fl / ms / 1e9, bn.peaks, us_per_launch=ms * 1e3, sequences=B)
    bn.be.synchronize()
    return roofline, other


# --------------------------------------------------------------------------- extra records
def extra_weak_dp(bn: Bench) -> dict:
    """32 sequences on EVERY rank (rank-specific prompts), the weak-scaling figure of the same job."""
    a = bn.a
    from kandle_b200 import synth
    from kandle_b200.core import Tensor
    eng, B, S, T = bn.engine, a.sequences, a.prompt, a.decode
    ids = Tensor(synth.token_ids(f"bench.ids.rank{bn.rank}", (B, S), a.vocab))
    bn.job_device(eng, ids, T)
    bn.sync_all()
    from kandle_b200.backend import CudaEvent
    e0, e1 = CudaEvent(), CudaEvent()
    e0.record()
    reps = 2
    for _ in range(reps):
        bn.job_device(eng, ids, T)
    e1.record()
    bn.sync_all()
    (ms,) = bn.max_over_ranks([e0.elapsed_ms(e1) / reps])
    ids.dispose()
    return {"scaling": "weak", "sequences_per_gpu": B, "tokens_per_s": B * (S + T) * bn.world / (ms * 1e-3), "ms_per_step": ms, "steps": reps}


def extra_tp_4b(bn: Bench) -> dict:
    """Config 4: Qwen3-4B shapes, 8 x 4096 prompt + 128 greedy steps, one model tensor-parallel over all ranks."""
    a = bn.a
    from kandle_b200 import core, lib, parallel, synth
    from kandle_b200.backend import CudaEvent
    from kandle_b200.core import Tensor
    world, rank = bn.world, bn.rank
    dims = dict(ARCH_4B)
    L = a.tp_layers
    if dims["kv_heads"] % world or dims["heads"] % world or dims["inter"] % (world * 16):
        return {"skipped": f"Qwen3-4B heads / MLP columns do not divide over {world} ranks"}
    if world > 1 and not bn.tp_ready:
        def bcast(obj):
            box = [obj]
            bn.dist.broadcast_object_list(box, src=0)
            return box[0]
        parallel.init_tensor_parallel(rank, world, bcast)

        def allgather(obj):
            out = [None] * world
            bn.dist.all_gather_object(out, obj)
            return out
        parallel.init_peer_buffers(rank, world, allgather)     # one-shot all-reduce of the decode step
        bn.tp_ready = True
    B, S, T = 8, 4096, 128
    eng = bn.make_engine(dims, L, dims["vocab"], B, S + T + 16, tp_size=world)
    ids = Tensor(synth.token_ids("bench.ids.tp", (B, S), dims["vocab"]))       # every rank the same batch
    bn.job_device(eng, ids, T)       # warm-up: graph capture, scratch sizes
    bn.sync_all()
    reps = 2
    e0, e1 = CudaEvent(), CudaEvent()
    e0.record()
    for _ in range(reps):
        bn.job_device(eng, ids, T)
    e1.record()
    bn.sync_all()
    ms = e0.elapsed_ms(e1) / reps
    p0, p1, p2 = CudaEvent(), CudaEvent(), CudaEvent()
    p0.record()
    tok = eng.prefill(ids)
    p1.record()
    eng.start_decode(tok, use_graph=True)
    for _ in range(1, T):
        eng.decode_step()
    p2.record()
    bn.be.synchronize()
    ms_prefill, ms_decode = p0.elapsed_ms(p1), p1.elapsed_ms(p2)
    rec = {}
    decode_kernels = ("separate kernels with all-reduces after o_proj and down_proj" if not eng._decode["fused"] else
                      "attention + one fused layer kernel per layer" if world == 1 else
                      "attention + one fused layer kernel per layer; the partial sums of o_proj and down_proj cross NVLink inside that kernel")
    if world > 1:
        # the collectives alone, on the buffers the engine reduces: 2 per layer, 72 per forward
        part = eng._bufs(B, S)["part"]
        d = eng._decode
        ms_ar_prefill = bn.timed_ms(lambda: eng._allreduce(part), reps=10, warm=2)
        ms_ar_o = bn.timed_ms(lambda: eng._allreduce(d["o_p"]), reps=50, warm=5)
        ms_ar_d = bn.timed_ms(lambda: eng._allreduce(d["down_p"]), reps=50, warm=5)
        bn.sync_all()
        # the fused one-shot kernel (sum over ranks through peer memory + residual add + RMSNorm) against
        # what it replaces (library all-reduce, then the add + RMSNorm kernel)
        lw0 = eng.layers[0]
        ms_fused = bn.timed_ms(lambda: eng._reduce_add_norm(d, d["o_p"], lw0["post_norm"], d["h"], d["h1"]), reps=50, warm=5)
        def unfused():
            eng._allreduce(d["o_p"])
            eng._norm(d["o_p"], lw0["post_norm"], d["x"], resid=d["h"], sum_out=d["h1"])
        ms_unfused = bn.timed_ms(unfused, reps=50, warm=5)
        # the decode phase again (new graphs): separate kernels with the one-shot all-reduce, then with
        # the library all-reduce
        def decode_again():
            eng.dispose()
            q0, q1 = CudaEvent(), CudaEvent()
            tok = eng.prefill(ids)
            eng.start_decode(tok, use_graph=True)
            q0.record()
            for _ in range(1, T):
                eng.decode_step()
            q1.record()
            bn.be.synchronize()
            bn.sync_all()
            return q0.elapsed_ms(q1)
        layer_kernel_in_use = bool(d["fused"])
        eng.use_fused_layer = False
        ms_decode_oneshot = decode_again()
        eng.use_p2p = False
        ms_decode_nccl = decode_again()
        eng.use_p2p = True
        eng.use_fused_layer = True
        bn.sync_all()
        ms_ar_prefill, ms_ar_o, ms_ar_d, ms_fused, ms_unfused, ms_decode_nccl, ms_decode_oneshot = bn.max_over_ranks(
            [ms_ar_prefill, ms_ar_o, ms_ar_d, ms_fused, ms_unfused, ms_decode_nccl, ms_decode_oneshot])
        nbytes = part.numel * 2
        rec["allreduce"] = {
            "library": "NCCL (ncclAllReduce on the library's stream)",
            "prefill_message_bytes": nbytes, "prefill_us_per_call": ms_ar_prefill * 1e3,
            "prefill_bus_gbs": 2.0 * (world - 1) / world * nbytes / (ms_ar_prefill * 1e-3) / 1e9,
            "prefill_ms_per_forward": ms_ar_prefill * 2 * L,
            "decode_message_bytes": [int(d["o_p"].numel * 4), int(d["down_p"].numel * 4)],
            "decode_us_per_call": [ms_ar_o * 1e3, ms_ar_d * 1e3],
            "decode_ms_per_step": (ms_ar_o + ms_ar_d) * L,
            "one_shot_peer_memory": {"kernel": "allreduce_add_rmsnorm_kernel (sum over ranks by peer loads + residual add + RMSNorm)",
                                     "us_per_call": ms_fused * 1e3, "replaces_us_per_call": ms_unfused * 1e3,
                                     "in_use": bool(d["p2p"]) and not layer_kernel_in_use},
            "decode_ms_per_step_by_variant": {
                "layer_kernel_with_in_kernel_exchange": layer_kernel_in_use,      # replaced by the time below
                "separate_kernels_one_shot_peer_memory": ms_decode_oneshot / (T - 1),
                "separate_kernels_library_allreduce": ms_decode_nccl / (T - 1)},
        }
    ms, ms_prefill, ms_decode = bn.max_over_ranks([ms, ms_prefill, ms_decode])
    if world > 1:
        v = rec["allreduce"]["decode_ms_per_step_by_variant"]
        v["layer_kernel_with_in_kernel_exchange"] = ms_decode / (T - 1) if v["layer_kernel_with_in_kernel_exchange"] else None
    per_layer_params = dims["hidden"] * ((dims["heads"] + 2 * dims["kv_heads"]) * dims["head_dim"]) + \
        dims["hidden"] * dims["heads"] * dims["head_dim"] + 3 * dims["hidden"] * dims["inter"]
    flops_prefill = B * S * (2.0 * per_layer_params * L) + 4.0 * B * dims["heads"] * dims["head_dim"] * (S * (S + 1) / 2) * L
    (_, _), (tc_peak, _) = bn.peaks
    rec.update({
        "workload": f"qwen3-4b-tp-bf16-b{B}-p{S}-d{T}" + ("" if L == ARCH_4B["layers"] else f"-L{L}"), "parallelism": f"tp{world}",
        "scaling": "strong", "lm_head": "tied to the embedding, replicated on every rank",
        "tokens_per_s": B * (S + T) / (ms * 1e-3), "ms_per_step": ms, "steps": reps,
        "prefill_ms": ms_prefill, "decode_ms_per_step": ms_decode / (T - 1),
        "prefill_tflops_per_gpu": flops_prefill / world / (ms_prefill * 1e-3) / 1e12,
        "prefill_frac_of_tensor_peak": flops_prefill / world / (ms_prefill * 1e-3) / 1e12 / tc_peak,
        "decode_kernels": decode_kernels,
    })
    eng.dispose()
    ids.dispose()
    del eng
    bn.release_memory()
    return rec


def extra_whisper_c5(bn: Bench) -> dict:
    """Config 5: Whisper-small encoder (bf16 fast path), 64 clips of 30 s (80 x 3000 log-mel) sharded over the ranks."""
    from kandle_b200 import core, lib, parallel, synth
    from kandle_b200.backend import CudaEvent
    from kandle_b200.core import Tensor
    from kandle_b200.model_utils import WhisperAudioEncoder, WhisperConfig
    from kandle_b200.whisper_engine import WhisperEncoderEngine
    clips_total, layers = 64, 12
    lo, hi = parallel.shard_range(clips_total, bn.rank, bn.world)
    n = hi - lo
    w = synth.whisper_encoder_weights(n_mels=80, state=768, layers=layers, n_ctx=1500, std=0.02)
    cfg = WhisperConfig(nMels=80, nAudioCtx=1500, nAudioState=768, nAudioHead=12, nAudioLayer=layers, dtype="bfloat16")
    enc = WhisperAudioEncoder(cfg)
    enc.loadStateDict(w)
    eng = WhisperEncoderEngine(enc)
    # log-mel stand-in with the value range of the real front end (clamped log10 spectrum scaled to about [-1, 1.5])
    rng = np.random.Generator(np.random.PCG64([1234, 5, bn.rank]))
    mel_host = lib.f32_to_bf16_bits(rng.uniform(-1.0, 1.5, size=(n, 80, 3000)).astype(np.float32))
    mel = core.empty((n, 80, 3000), "bfloat16")
    bn.be.upload(mel._handle, mel_host)
    pinned = ctypes.c_void_p()
    lib.call("kd_host_alloc_pinned", ctypes.c_uint64(mel_host.nbytes), ctypes.byref(pinned))
    ctypes.memmove(pinned, mel_host.ctypes.data, mel_host.nbytes)
    out_bytes = n * 1500 * 768 * 2
    out_pinned = ctypes.c_void_p()
    lib.call("kd_host_alloc_pinned", ctypes.c_uint64(out_bytes), ctypes.byref(out_pinned))
    for _ in range(2):
        eng.forward(mel).dispose()
    bn.sync_all()
    reps = 5
    e0, e1 = CudaEvent(), CudaEvent()
    e0.record()
    for _ in range(reps):
        eng.forward(mel).dispose()
    e1.record()
    bn.sync_all()
    ms = e0.elapsed_ms(e1) / reps
    t0 = time.perf_counter()
    for _ in range(reps):
        lib.call("kd_upload_async", ctypes.c_uint64(mel._handle.storage.handle), ctypes.c_uint64(0), pinned, ctypes.c_uint64(mel_host.nbytes))
        y = eng.forward(mel)
        lib.call("kd_download_async", ctypes.c_uint64(y._handle.storage.handle), ctypes.c_uint64(0), out_pinned, ctypes.c_uint64(out_bytes))
        bn.be.synchronize()
        y.dispose()
    bn.sync_all()
    ms_e2e = (time.perf_counter() - t0) * 1e3 / reps
    ms, ms_e2e = bn.max_over_ranks([ms, ms_e2e])
    flops = clips_total * (6.4e9 + layers * 28.15e9)        # 344.2 GFLOP per clip
    (_, _), (tc_peak, _) = bn.peaks
    for p in (pinned, out_pinned):
        lib.call("kd_host_free_pinned", p)
    mel.dispose()
    del eng, enc
    bn.release_memory()
    return {"workload": "whisper-small-encoder-bf16-64clips", "parallelism": f"dp{bn.world}", "scaling": "strong", "clips_per_gpu": n,
            "clips_per_s": clips_total / (ms * 1e-3), "ms_per_step": ms, "steps": reps,
            "tflops_per_gpu": flops / bn.world / (ms * 1e-3) / 1e12, "frac_of_tensor_peak": flops / bn.world / (ms * 1e-3) / 1e12 / tc_peak,
            "frac_of_nominal_tensor_peak": flops / bn.world / (ms * 1e-3) / 1e12 / NOMINAL_BF16_TFLOPS,
            "e2e_clips_per_s": clips_total / (ms_e2e * 1e-3), "e2e_h2d_bytes_per_step": int(mel_host.nbytes) * bn.world,
            "e2e_d2h_bytes_per_step": int(out_bytes) * bn.world}


def run_ours(a) -> None:
    bn = Bench(a)
    from kandle_b200 import lib
    line = run_headline(bn)
    extras = [] if a.no_extras else [e for e in a.extras.split(",") if e]
    if "weak_dp" in extras and bn.world > 1:
        line["weak_dp"] = extra_weak_dp(bn)
    bn.engine.dispose()
    bn.engine = None
    bn.release_memory()
    for name, fn in (("whisper_c5", extra_whisper_c5), ("tp_4b", extra_tp_4b)):
        if name in extras:
            try:
                line[name] = fn(bn)
            except Exception as e:  # an extra record must not take the headline down with it
                line[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if bn.rank == 0 and bn.world == 1 and not a.no_cpu_baseline:
        v, desc, threads, _ = cpu_arm(a.cpu_sample, a.layers, a.vocab)
        line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc}
    else:
        line["cpu_baseline"] = None
    if bn.rank == 0:
        print(json.dumps(line), flush=True)
    if bn.tp_ready:
        lib.call("kd_p2p_disconnect")
        lib.call("kd_comm_destroy")
    if bn.dist is not None:
        bn.dist.barrier()
        bn.dist.destroy_process_group()


def main():
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
