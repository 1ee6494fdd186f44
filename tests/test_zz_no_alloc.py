"""GPU: the split-K GEMV that carries its own scratch memory.

Callers that are not allowed to allocate on the device (an executor whose
arenas are frozen after start-up, a step replayed from a CUDA graph, a plugin
host that offers no allocator) use mc_sm100_decode_gemv_splitk_static.  It must
return what the regular split-K call returns with a caller-provided partial
buffer.  The two calls below run back to back on the same built-in array, the
second with a different shape and split, so anything the first call left behind
would show.  The file name sorts last on purpose: a run that stops at the first
failure has then already run every other test."""
import numpy as np
import pytest

import oracle_np as onp
from parity import check_close

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_static_scratch_matches_caller_scratch_twice(pkg):
    assert torch.cuda.is_available()
    import gpu_util as g
    for N, K, S in ((2304, 5760, 8), (3456, 2304, 2)):
        w = onp.seeded_bf16(900 + N, (N, K), 0.02)
        x = onp.seeded_bf16(901 + N, (K,), 1.0)
        dw, dx = g.dev(w), g.dev(x)
        y_ref, y_new = g.empty_u16(N), g.empty_u16(N)
        part = torch.empty(S * N, dtype=torch.float32, device="cuda")
        pkg.launch_decode_gemv(dw, dx, y_ref, N, K, pkg.TACTIC_SPLITK, S, part)
        pkg.launch_decode_gemv_splitk_static(dw, dx, y_new, N, K, S)
        g.sync()
        # same kernels, same fixed-order merge: the two results are the same bits
        assert np.array_equal(g.host_u16(y_new), g.host_u16(y_ref)), f"static vs caller scratch N={N} K={K} S={S}"
        check_close(g.host_u16(y_new), onp.linear_bf16(w, x), what=f"static scratch vs oracle N={N}")


def test_static_scratch_rejects_oversize(pkg):
    w = torch.zeros(16, dtype=torch.int16, device="cuda")
    with pytest.raises(pkg.McError) as e:
        pkg.launch_decode_gemv_splitk_static(w, w, w, 131072, 64, 2)      # 2 * 131072 floats > built-in array
    assert e.value.status == pkg.MC_E_UNSUPPORTED and "exceeds" in e.value.message
