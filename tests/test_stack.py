"""The decode stack object: arena layout on CPU, the whole chain against the oracle on GPU."""
import numpy as np
import pytest

import oracle_np as onp
from parity import check_close


def test_stack_layout_and_validation(pkg):
    d = pkg.stack_desc(3, 256, 384, 512, 1000, fp8=True, max_batch=8)
    wbytes, sbytes = pkg.stack_sizes(d)
    seen = []
    for l in range(3):
        for name in ("qkv", "o", "gate_up", "down", "norm1", "norm2", "qkv_scale", "o_scale", "gate_up_scale", "down_scale"):
            off, n = pkg.stack_section(d, l, name)
            assert off % 256 == 0 and n > 0
            seen.append((off, n))
    for name in ("lm_head", "final_norm", "lm_head_scale"):
        seen.append(pkg.stack_section(d, 0, name))
    seen.sort()
    assert all(a[0] + a[1] <= b[0] for a, b in zip(seen, seen[1:])), "sections overlap"
    assert seen[-1][0] + seen[-1][1] <= wbytes and sbytes > 0
    assert pkg.stack_section(d, 1, "gate_up")[1] == 2 * 512 * 256            # e4m3: one byte per weight
    assert pkg.stack_section(pkg.stack_desc(3, 256, 384, 512, 1000), 0, "qkv_scale")[1] == 0   # bf16: no scales
    bad = pkg.stack_desc(3, 256, 384, 512, 1000)
    bad.struct_size = 12
    with pytest.raises(pkg.McError):
        pkg.stack_sizes(bad)
    bad = pkg.stack_desc(3, 250, 384, 512, 1000)                             # hidden not a multiple of 8
    with pytest.raises(pkg.McError):
        pkg.stack_sizes(bad)
    bad = pkg.stack_desc(3, 256, 384, 512, 1000, max_batch=65)
    with pytest.raises(pkg.McError):
        pkg.stack_sizes(bad)


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("M", [1, 3, 8, 16])
def test_stack_matches_oracle_chain(pkg, fp8, M):
    torch = pytest.importorskip("torch")
    import stack_util as su
    layers, H, Q, I, V = 3, 512, 768, 1024, 4099
    w = su.make_weights(layers, H, Q, I, V)
    desc = pkg.stack_desc(layers, H, Q, I, V, fp8=fp8, max_batch=16)
    arena, scratch = su.upload(pkg, torch, desc, w, fp8)
    st = pkg.stack_create(desc, arena, scratch)
    try:
        x = onp.seeded_bf16(700 + M, (M, H), 1.0)
        hx = torch.from_numpy(x.view(np.int16)).pin_memory()
        htok = torch.full((M,), -1, dtype=torch.int32).pin_memory()
        stream = torch.cuda.Stream()
        toks = []
        for _ in range(3):                          # eager, capture, replay: identical tokens
            pkg.stack_step_host(st, hx, M, htok, stream)
            toks.append(htok.clone())
        assert all(torch.equal(toks[0], t) for t in toks[1:])
        ref = su.oracle_stack(w, x if M > 1 else x[0], fp8).reshape(M, V)
        logits_dev = torch.empty((M, V), dtype=torch.int16, device="cuda")
        import ctypes
        src = pkg.stack_logits_ptr(st)
        assert torch.cuda.current_device() == 0 and src
        ctypes.CDLL("libcudart.so").cudaMemcpy(ctypes.c_void_p(logits_dev.data_ptr()), ctypes.c_void_p(src),
                                                ctypes.c_size_t(M * V * 2), 3)
        got = logits_dev.cpu().numpy().view(np.uint16)
        # three layers of bf16-rounded intermediates: a flipped last bit upstream moves the logits a little
        gf, rf = onp.bf16_to_f32(got).astype(np.float64), onp.bf16_to_f32(ref).astype(np.float64)
        rel = np.sqrt(((gf - rf) ** 2).sum() / (rf ** 2).sum())
        assert rel < 1e-2, rel
        cos = (gf * rf).sum() / np.sqrt((gf ** 2).sum() * (rf ** 2).sum())
        assert cos > 0.9999
        for m in range(M):
            top = np.sort(rf[m])[-2:]
            if top[1] - top[0] > 0.05:
                assert int(toks[0][m]) == int(np.argmax(rf[m]))
            assert int(toks[0][m]) == onp.greedy(got[m])
    finally:
        pkg.stack_destroy(st)
