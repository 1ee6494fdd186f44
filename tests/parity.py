"""Tolerance set shared by the parity tests.

The reference budgets, for a GEMV against a CPU statement with a different
accumulation order: relative L2 error < 1e-2 and every element within 2 bf16
units in the last place (native/tests/gemv_bench.cpp:5-7, 140-161), plus an
absolute floor of 1e-3 (bf16) / 1e-4 (fp8) for results that cancel to nearly
zero (native/tests/kernel_ops.cpp:867-885).  On top of that the maximum
relative error over elements that are not tiny (|ref| >= 2^-7 * rms) must stay
within 1e-2.
"""
import numpy as np

import oracle_np as onp

REL_L2_MAX = 1e-2
ULP_MAX = 2
REL_ERR_MAX = 1e-2


def check_close(got_u16, ref_u16, abs_floor=1e-3, what="", rel_max=REL_ERR_MAX):
    got = onp.bf16_to_f32(np.asarray(got_u16).reshape(-1)).astype(np.float64)
    ref = onp.bf16_to_f32(np.asarray(ref_u16).reshape(-1)).astype(np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    d = np.abs(got - ref)
    rel_l2 = np.sqrt((d ** 2).sum() / max((ref ** 2).sum(), 1e-30))
    ulp = onp.bf16_ulp(ref.astype(np.float32)).astype(np.float64)
    bad = d > ULP_MAX * ulp + abs_floor
    rms = np.sqrt((ref ** 2).mean())
    big = np.abs(ref) >= rms * 2.0 ** -7
    max_rel = float((d[big] / np.abs(ref[big])).max()) if big.any() else 0.0
    exact = float((d == 0).mean())
    msg = (f"{what}: relL2={rel_l2:.3e} maxulp={(d / ulp).max():.2f} maxrel={max_rel:.3e} "
           f"exact={exact:.4f} bad={int(bad.sum())}")
    assert rel_l2 <= REL_L2_MAX, msg
    assert not bad.any(), msg
    assert max_rel <= rel_max, msg
    return {"rel_l2": rel_l2, "max_rel": max_rel, "exact": exact}
