"""Host logic of two launch plans, checked without a GPU through the library's host-only views: how the
register-streaming batched GEMM cuts a weight into row blocks, and what the persistent M = 1 kernel's
shared-memory ring looks like for a given stack (or that it does not fit and the per-linear kernels run)."""
import pytest


@pytest.mark.parametrize("n,sms,want", [
    (2304, 148, (16, 1, 16)),        # o_proj / down_proj: one 16-row block per CTA
    (3456, 148, (8, 3, 24)),         # qkv: 8-row blocks spread 23.4 rows per SM more evenly than 16-row ones (32 on the fullest)
    (11520, 148, (16, 5, 80)),       # gate_up: five blocks per CTA at a time
    (122753, 148, (16, 16, 832)),    # lm_head: a warp owns whole blocks
    (1152, 148, (8, 1, 8)),          # a half-width shard: 144 CTAs of 8 rows instead of 72 of 16
    (100, 148, (8, 1, 8)),
    (2304, 132, (8, 3, 24)),         # fewer SMs: 2304 / 132 = 17.5 rows per SM
])
def test_mma_rows_plan(pkg, n, sms, want):
    rows, r, worst = pkg.debug_mma_rows_plan(n, sms)
    assert (rows, r, worst) == want
    blocks = (n + rows - 1) // rows
    grid = min(blocks, sms)
    assert r * 1 <= 16 and worst == ((blocks + grid - 1) // grid) * rows
    # never worse than the other block height
    other = 8 if rows == 16 else 16
    ob = (n + other - 1) // other
    assert worst <= ((ob + min(ob, sms) - 1) // min(ob, sms)) * other


@pytest.mark.parametrize("fp8", [False, True])
def test_chain_plan(pkg, fp8):
    wb = 1 if fp8 else 2
    slot, rows_h, rows_gu, rows_dn = pkg.debug_chain_plan(fp8, 2304, 5760)
    # 16 slots + both copies of the widest activation + the residual fit 227 KB, slots are 128-byte multiples
    assert slot % 128 == 0 and 16 * slot + 5760 * 2 * (2 if fp8 else 1) + 2304 * 2 + 1024 + 128 <= 227 * 1024
    assert rows_h == min(32, slot // (2304 * wb)) and rows_dn == min(32, slot // (5760 * wb))
    assert rows_gu % 2 == 0 and rows_gu in (rows_h, rows_h - 1)           # whole gate/up pairs
    assert rows_h * 2304 * wb <= slot and rows_dn >= 1
    # the benchmark's stack: units of 9 - 12 KB (the copy engine takes ~0.2 us per request whatever its size)
    assert 9 * 1024 <= rows_h * 2304 * wb <= 12 * 1024 + 512
    # a stack whose rows do not fit a slot: the kernel is not used
    assert pkg.debug_chain_plan(fp8, 8192, 28672)[0] == 0
    assert pkg.debug_chain_plan(fp8, 65536, 65536) == (0, 0, 0, 0)
    # a small stack: row scales travel one per lane, so a slot never holds more than 32 rows
    s2, h2, g2, d2 = pkg.debug_chain_plan(fp8, 256, 512)
    assert s2 > 0 and h2 <= 32 and g2 <= 32 and d2 <= 32 and g2 % 2 == 0
