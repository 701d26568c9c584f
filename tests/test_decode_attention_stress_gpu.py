"""Fresh-process stress of the split-KV decode attention.

One recorded failure of this kernel happened in the first process on a machine, on a ragged shape
(last key tile holding one key, nine splits), and never again in a warm process.  The protocol hole
that fits it (the wait for the last P V product could pass two mbarrier phases early when the tensor
pipe lagged behind the softmax warps) only opens under unusual timing, which a cold process is most
likely to produce: cold instruction caches, cold TLBs, first use of the scratch buffer.  So the
ragged cases run here in several new processes, each starting with a different case, with the
library's scratch and the output poisoned with NaN patterns before every launch."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("rotation", range(6))
def test_ragged_decode_attention_as_first_launch_of_a_fresh_process(rotation):
    r = subprocess.run([sys.executable, os.path.join(HERE, "decode_attention_cases.py"), str(rotation)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, f"rotation {rotation} failed:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    assert "ragged cases ok" in r.stdout
