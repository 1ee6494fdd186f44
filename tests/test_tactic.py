"""Tactic selection of the M = 1 bf16 GEMV: the static split rule on CPU, timing-based selection on GPU."""
import numpy as np
import pytest

import oracle_np as onp
from parity import check_close


def test_partial_size_rule(pkg):
    assert pkg.lib().mc_sm100_gemv_partial_floats(3456) == 8 * 3456       # 8 segments at most (gemv_tactic.h:43, 58-64)


@pytest.mark.gpu
def test_static_split_rule(pkg):
    """gemv_tactic.h:42-56 with the block target of this device (two CTAs' worth per SM): large N is never split,
    small N takes the largest of 8 / 4 / 2 that divides K into multiples of 8 and reaches the target."""
    lib = pkg.lib()
    sms = pkg.device_check()["sm_count"]
    assert lib.mc_sm100_gemv_pick_split_s(122753, 2304) == 1              # N > 4096
    assert lib.mc_sm100_gemv_pick_split_s(8 * 2 * sms, 2304) == 1         # already enough blocks
    s = lib.mc_sm100_gemv_pick_split_s(2304, 2304)
    assert s in (1, 2, 4, 8) and (s == 1 or (2304 // 8) * s >= 2 * sms)
    n = 8 * ((2 * sms + 7) // 8)                                          # n / 8 blocks: an eight-way split just reaches the target
    assert lib.mc_sm100_gemv_pick_split_s(n, 2304) == 8
    assert lib.mc_sm100_gemv_pick_split_s(n, 2296) == 1                   # no split leaves segments that are multiples of 8
    assert lib.mc_sm100_gemv_pick_split_s(64, 2304) == 1                  # even eight segments do not reach the target: not split


@pytest.mark.gpu
@pytest.mark.parametrize("N,K", [(2304, 2304), (2304, 5760), (64, 4096), (8192, 2304)])
def test_selected_tactic_runs_and_matches_oracle(pkg, N, K):
    torch = pytest.importorskip("torch")
    import gpu_util as g
    w = onp.seeded_bf16(300 + N + K, (N, K), 0.02)
    x = onp.seeded_bf16(301 + N + K, (K,), 1.0)
    dw, dx, dy = g.dev(w), g.dev(x), g.empty_u16(N)
    nf = pkg.lib().mc_sm100_gemv_partial_floats(N)
    part = torch.empty(nf, dtype=torch.float32, device="cuda")
    flush = torch.empty(300 << 20, dtype=torch.uint8, device="cuda")
    for fl in (None, flush):
        t = pkg.select_decode_gemv_tactic(dw, N, K, dx, dy, part, nf, fl)
        assert t.tactic in (pkg.TACTIC_ROWS, pkg.TACTIC_SPLITK) and t.us_rows > 0
        if N > 4096:
            assert t.tactic == pkg.TACTIC_ROWS and t.us_splitk == 0          # split-K is not a candidate for large N
        else:
            assert t.us_splitk > 0 and t.best_split_s in (2, 4, 8)
            if t.tactic == pkg.TACTIC_SPLITK:
                assert t.us_splitk < t.us_rows and t.split_s == t.best_split_s
        dy = g.empty_u16(N)                                              # poisoned with NaN: every element must be written
        pkg.run_decode_gemv(t, dw, dx, dy, N, K, part)
        g.sync()
        check_close(g.host_u16(dy), onp.linear_bf16(w, x), what=f"selected tactic {t.tactic}/{t.split_s} N={N} K={K}")
