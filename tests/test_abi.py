"""CPU checks of the boundary: the shared library loads without a GPU, exports every symbol the
header declares, reports errors instead of computing when no device is initialised, and the
host-side view arithmetic (slices, permutes, broadcast) matches numpy."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"\bint\s+(kd_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_entry_points():
    names = _declared_symbols()
    assert "kd_flash_attention" in names and "kd_matmul" in names and len(names) >= 30


def test_library_loads_and_exports_every_declared_symbol():
    from kandle_b200 import lib
    so = ctypes.CDLL(lib.LIB_PATH)
    missing = [n for n in _declared_symbols() if not hasattr(so, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_python_binding_covers_every_declared_symbol():
    from kandle_b200 import lib
    missing = [n for n in _declared_symbols() if n not in lib._SIGNATURES and n not in lib.EXTRA_SIGNATURES]
    assert not missing, missing


def test_calls_fail_loudly_without_init():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the not-initialised path is covered on CPU boxes")
    from kandle_b200 import lib
    with pytest.raises(lib.KandleCudaError) as e:
        lib.call("kd_synchronize")
    assert e.value.status == 4
    with pytest.raises(lib.KandleCudaError) as e:
        lib.call("kd_init", 0, 0)
    assert "no CPU fallback" in str(e.value)


def test_struct_layout_matches_header():
    from kandle_b200 import lib
    assert ctypes.sizeof(lib.kd_tensor) == 8 + 8 + 4 + 4 + 8 * 8 * 2
    assert ctypes.sizeof(lib.kd_matmul_cfg) == 3 * 8 + 2 * 4 + 2 * 4 + 2 * 4


def test_bf16_host_conversion_round_to_nearest_even():
    from kandle_b200 import lib
    import torch
    x = np.random.default_rng(0).standard_normal(10000).astype(np.float32) * 100
    x[:4] = [0.0, -0.0, np.inf, 1.00390625]  # last one is an exact tie
    bits = lib.f32_to_bf16_bits(x)
    t = torch.tensor(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, t)
    assert np.array_equal(lib.bf16_bits_to_f32(bits), torch.tensor(x).to(torch.bfloat16).float().numpy())


def test_slice_parser_and_broadcast():
    from kandle_b200 import core
    items = core._parse_slice("..., :64", (2, 3, 128))
    assert items == [slice(None), slice(None), slice(None, 64)]
    items = core._parse_slice(":, :, 3:7, :", (1, 2, 10, 4))
    assert items[2] == slice(3, 7)
    assert core._broadcast_shape((4, 1, 3), (5, 1)) == (4, 5, 3)
    with pytest.raises(ValueError):
        core._broadcast_shape((4, 3), (5,))
    assert core._promote("int32", "float32") == "float32"
    assert core._promote("bfloat16", "float32") == "float32"


class _FakeStorage:
    """Stands in for a device storage so that view arithmetic can be checked without a GPU."""
    handle, id, nbytes = 1, 1, 1 << 20

    def incRef(self):
        pass

    def decRef(self):
        pass

    isDisposed = False


def test_select_and_integer_index_raise_like_the_reference():
    """packages/core/src/dispatch/handlers/shape.ts:500-518: a dim or an index outside its range is an
    error, never a wrap-around to another element."""
    from kandle_b200 import core
    from kandle_b200.backend import CudaTensorHandle
    t = core.Tensor(_handle=CudaTensorHandle(_FakeStorage(), (4, 5, 6), "float32"))
    assert t.select(1, -1).shape == (4, 6) and t.select(1, -1).offset == 4 * 6
    assert t.select(-1, 2).shape == (4, 5) and t.select(-1, 2).offset == 2
    with pytest.raises(IndexError, match="index 5 out of range for dim 1 with size 5"):
        t.select(1, 5)
    with pytest.raises(IndexError, match="index -6 out of range"):
        t.select(1, -6)
    with pytest.raises(IndexError, match="dim 3 out of range for tensor with 3 dimensions"):
        t.select(3, 0)
    with pytest.raises(IndexError):
        t.slice(":, 7, :")
    assert t.slice(":, -5, 1:3").shape == (4, 2)
