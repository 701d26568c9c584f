"""Multi-GPU helpers: one process (rank) per GPU.

Two ways the hot path spreads over GPUs:
  * independent sequences / clips are sharded across ranks with replicated weights and no data-path
    collective (`shard_range`);
  * a model too large or too slow for one GPU is tensor-parallel: attention heads and MLP columns are
    split across ranks (`shard_qwen3_weights`) and the partial outputs of o_proj and down_proj are
    summed with an NCCL all-reduce issued by the library on its own stream (`allreduce`).
The reference has neither (it is single-device); N-GPU results are checked against 1-GPU results.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import lib


def shard_range(n_items: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of the items rank `rank` owns; the first n_items % world ranks get one extra."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_items, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_qwen3_weights(weights: dict, *, heads: int, kv_heads: int, head_dim: int, rank: int, world: int) -> dict:
    """Tensor-parallel slice of HuggingFace-style Qwen3 weights for one rank: q/k/v projections by
    head (output rows), o_proj by the matching input columns, gate/up by intermediate rows, down by
    the matching input columns; norms and the embedding / tied lm_head are replicated."""
    if heads % world or kv_heads % world:
        raise ValueError(f"{heads} query / {kv_heads} kv heads do not divide over {world} ranks")
    out = {}
    hq, hkv = heads // world, kv_heads // world
    for name, w in weights.items():
        if name.endswith("q_proj.weight"):
            out[name] = w[rank * hq * head_dim:(rank + 1) * hq * head_dim]
        elif name.endswith("k_proj.weight") or name.endswith("v_proj.weight"):
            out[name] = w[rank * hkv * head_dim:(rank + 1) * hkv * head_dim]
        elif name.endswith("o_proj.weight"):
            out[name] = w[:, rank * hq * head_dim:(rank + 1) * hq * head_dim]
        elif name.endswith("gate_proj.weight") or name.endswith("up_proj.weight"):
            inter = w.shape[0]
            if inter % world:
                raise ValueError(f"intermediate size {inter} does not divide over {world} ranks")
            out[name] = w[rank * inter // world:(rank + 1) * inter // world]
        elif name.endswith("down_proj.weight"):
            inter = w.shape[1]
            out[name] = w[:, rank * inter // world:(rank + 1) * inter // world]
        else:
            out[name] = w
    return {k: np.ascontiguousarray(v) for k, v in out.items()}


def default_nccl_path() -> str:
    """Prefer the NCCL that ships with torch's CUDA wheels when present, else the system library."""
    try:
        import nvidia.nccl  # type: ignore
        p = os.path.join(os.path.dirname(nvidia.nccl.__file__), "lib", "libnccl.so.2")
        if os.path.exists(p):
            return p
    except Exception:
        pass
    return ""


def init_tensor_parallel(rank: int, world: int, broadcast) -> None:
    """Creates the library's NCCL communicator.  `broadcast(obj_or_None) -> obj` must return rank 0's
    object on every rank (e.g. a torch.distributed.broadcast_object_list wrapper)."""
    path = default_nccl_path().encode()
    ident = None
    if rank == 0:
        buf = ctypes.create_string_buffer(128)
        lib.call("kd_comm_unique_id", path, buf, 128)
        ident = buf.raw
    ident = broadcast(ident)
    lib.call("kd_comm_init", path, world, rank, ident, len(ident))


def allreduce(t) -> None:
    """In-place sum over ranks of a contiguous bf16/fp32 device tensor, on the library's stream."""
    lib.call("kd_allreduce_sum", ctypes.byref(t._handle.c()))


def init_peer_buffers(rank: int, world: int, allgather) -> None:
    """Maps every rank's peer buffer for the one-shot all-reduce (kd_allreduce_add_rmsnorm).
    `allgather(bytes) -> list[bytes]` must return every rank's object in rank order (e.g. a
    torch.distributed.all_gather_object wrapper).  All ranks must be on one node with peer access."""
    buf = ctypes.create_string_buffer(64)
    lib.call("kd_p2p_prepare", buf, 64)
    handles = allgather(buf.raw)
    if len(handles) != world:
        raise ValueError(f"expected {world} handles, got {len(handles)}")
    lib.call("kd_p2p_connect", world, rank, b"".join(handles), 64)


def peer_buffers_ready() -> bool:
    r = ctypes.c_int(0)
    lib.call("kd_p2p_info", ctypes.byref(r), None, None)
    return bool(r.value)
