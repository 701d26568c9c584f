"""The launch plan of the fused decode layer kernel, checked without a GPU over many shapes.

The kernel's CTAs wait for one another: a plan with an empty K range, a K range that starts in the
middle of a group of k-blocks, more slices than groups of CTAs, or partial sums that do not fit the
leader's shared memory would end in a bounded wait running out on the device.  The planner is pure
host arithmetic (kd_debug_decode_layer_plan), so its guarantees are fuzzed here."""
import ctypes
import itertools

import pytest

from kandle_b200 import lib

RED_BYTES = 24 * 1024
X_AREA, W_AREA = 16 * 1024, 32 * 1024


def _plan(seqs, hidden, attn, inter, qkv, tp, grids=(148, 148, 132)):
    out = (ctypes.c_int * 29)()
    lib.call("kd_debug_decode_layer_plan", seqs, hidden, attn, inter, qkv, tp, grids[0], grids[1], grids[2], out, 29)
    cluster = out[0]
    phases = [dict(zip(("N", "K", "n_unit", "units", "split", "kb_per", "kg"), out[1 + 7 * i: 8 + 7 * i])) for i in range(4)]
    return cluster, phases


def _check(seqs, cluster, phases, n_gemms, tp, grids):
    assert cluster in (1, 2, 4)
    G = {1: grids[0], 2: grids[1], 4: grids[2]}[cluster]
    assert G > 0 and seqs <= G
    if tp:
        assert cluster == 1
    x_box = 8 if seqs <= 8 else 16 if seqs <= 16 else 32 if seqs <= 32 else 64 if seqs <= 64 else 128
    for i, ph in enumerate(phases[:n_gemms]):
        n_kb = -(-ph["K"] // 64)
        assert 16 <= ph["n_unit"] <= 128 and ph["n_unit"] % (32 if i == 1 else 16) == 0
        assert ph["units"] == -(-ph["N"] // ph["n_unit"]) and 1 <= ph["units"] <= 512
        assert ph["split"] in (1, 2, 4) and cluster % ph["split"] == 0
        assert ph["kg"] >= 1 and ph["kg"] * x_box * 128 <= X_AREA and ph["kg"] * ph["n_unit"] * 128 <= W_AREA
        if i in (1, 3):
            assert ph["split"] == 1
        if i == 3:
            assert ph["n_unit"] == 128
        if ph["split"] == 1:
            assert ph["kb_per"] == n_kb
        else:
            S = ph["split"]
            assert ph["K"] % 64 == 0
            assert ph["kb_per"] % 2 == 0 and ph["kb_per"] % ph["kg"] == 0       # ranges start at even k-blocks and whole groups
            assert ph["kb_per"] * (S - 1) < n_kb <= ph["kb_per"] * S            # nobody's range is empty, all of K is covered
            assert ph["units"] <= G // S                                        # one wave of groups
            assert (S - 1) * seqs * ph["n_unit"] * 4 <= RED_BYTES               # partial sums fit the leader's shared memory
        if tp and i in (0, 2):
            assert ph["n_unit"] & (ph["n_unit"] - 1) == 0 and ph["units"] <= 128


def test_plans_of_the_configurations_that_are_measured():
    c, ph = _plan(32, 1024, 2048, 3072, 4096, 0)                  # Qwen3-0.6B layer, 32 sequences
    _check(32, c, ph, 4, 0, (148, 148, 132))
    assert c == 4 and ph[0]["split"] > 1 and ph[2]["split"] == 4 and ph[2]["n_unit"] == 32
    c, ph = _plan(8, 2560, 4096, 9728, 6144, 0)                   # Qwen3-4B layer, 8 sequences
    _check(8, c, ph, 4, 0, (148, 148, 132))
    assert c in (2, 4) and ph[0]["split"] == 2 and ph[2]["split"] == 2
    c, ph = _plan(8, 2560, 1024, 2432, 1536, 1)                   # one rank of four of the same layer
    _check(8, c, ph, 4, 1, (148, 148, 132))
    c, ph = _plan(48, 512, 320, 1056, 0, 0)                       # last layer form, K not a multiple of 64
    _check(48, c, ph, 3, 0, (148, 148, 132))
    assert ph[0]["split"] == 1 and ph[2]["split"] == 1            # ungrouped k-blocks are never split


@pytest.mark.parametrize("grids", [(148, 148, 132), (148, 0, 0), (132, 132, 120), (64, 64, 64), (148, 148, 0)])
def test_every_plan_keeps_the_kernels_preconditions(grids):
    seqs_list = [1, 4, 8, 9, 16, 31, 32, 33, 64, 100, 128]
    hidden_list = [256, 1024, 1536, 2560, 4096, 5120, 8192]
    n = 0
    for seqs, hidden, tp in itertools.product(seqs_list, hidden_list, (0, 1)):
        for attn, inter, qkv in ((hidden * 2, hidden * 3, 4096), (hidden, 11008, 128 * 6), (320, 1056, 0), (128, 512, 384),
                                 (hidden * 2 - 64, hidden * 3 + 32, 2048)):
            if seqs > max(grids):
                continue
            c, ph = _plan(seqs, hidden, attn, inter, qkv, tp, grids)
            if c == 0:
                continue                      # refused: the entry point reports "no launch configuration"
            _check(seqs, c, ph, 4 if qkv else 3, tp, grids)
            n += 1
    assert n > 400


def test_no_configuration_is_reported_as_such():
    c, _ = _plan(32, 1024, 2048, 3072, 4096, 0, grids=(0, 0, 0))
    assert c == 0
    c, _ = _plan(128, 1024, 2048, 3072, 4096, 0, grids=(64, 64, 64))          # more sequences than CTAs
    assert c == 0
