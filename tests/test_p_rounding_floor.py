"""Where the default path's residual error comes from, shown on the CPU.

oracle/emulate_p.py restates the one place where the sm_100a kernel departs from exact attention over the same
fp16-dequantised records: the softmax probabilities are rounded to fp16 before the P.V product (as in the reference
kernel, engine/attn.cu:261-263), under a reference exponent that follows the row maximum lazily (engine/attn.cu:237-255).
With that single rounding switched off the emulation agrees with the fp64 oracle to 1e-5 x output RMS; with it the
worst element sits between 1e-3 and 4e-3 x RMS from 2 K tokens on, which is the size of error the GPU tests measure on
the default path; carried as fp16 value + fp16 remainder it is back at 1e-5. So the stated bar (2e-3 x RMS) is a
statement about the precision P is carried in, and LLATTN_IO_PRECISE_P is the path that meets it at every length
(tests/test_gpu_precise.py; the GPU test there also checks the kernel against this emulation element by element)."""
import importlib

import numpy as np
import pytest


@pytest.fixture(scope="module")
def emu():
    import emulate_p
    return emulate_p


@pytest.mark.parametrize("nblocks", [64, 256])
def test_fp16_rounding_of_p_is_the_floor(orc, emu, pkg, nblocks):
    wl = pkg.workload
    Kc, Vc = wl.context_blocks(nblocks, seq=77)
    Q, Kf, Vf = wl.query_blocks(1, seq=77)
    cache = np.zeros((4, nblocks + 1, orc.REC_BYTES), np.uint8)
    orc.kv_commit(Kc, Vc, cache, nblocks + 1, 0)
    O1, _ = orc.attention(Q, Kf, Vf, cache, nblocks + 1, nblocks, dq_mode=1)
    rms = np.sqrt((O1.astype(np.float64) ** 2).mean())
    err = {m: np.abs(emu.attention_rounded_p(Q, Kf, Vf, cache, nblocks + 1, nblocks, m) - O1).max() / rms
           for m in ("fp32", "fp16x2", "fp16")}
    assert err["fp32"] <= 2e-5          # the emulation is the oracle's arithmetic when nothing is rounded
    assert err["fp16x2"] <= 5e-5        # value + remainder: as good as unrounded at the bar's scale
    assert 1e-3 <= err["fp16"] <= 4e-3  # one fp16 rounding of P: the default path's error, around the 2e-3 bar


def test_short_context_meets_the_bar_with_fp16_p(orc, emu, pkg):
    """Up to a few hundred keys the rows are not yet averaged down (RMS is large) and fp16 P is inside the bar."""
    wl = pkg.workload
    Kc, Vc = wl.context_blocks(8, seq=78)
    Q, Kf, Vf = wl.query_blocks(1, seq=78)
    cache = np.zeros((4, 9, orc.REC_BYTES), np.uint8)
    orc.kv_commit(Kc, Vc, cache, 9, 0)
    O1, _ = orc.attention(Q, Kf, Vf, cache, 9, 8, dq_mode=1)
    rms = np.sqrt((O1.astype(np.float64) ** 2).mean())
    assert np.abs(emu.attention_rounded_p(Q, Kf, Vf, cache, 9, 8, "fp16") - O1).max() / rms <= 2e-3
