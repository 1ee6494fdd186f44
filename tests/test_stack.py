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


# ---- the stack at the dimensions of the 40-layer benchmark workload ----------------------------
_FULL = {}


def _full_weights(pkg, fp8):
    """Two layers + lm_head at hidden 2304 / qkv 3456 / inter 5760 / vocab 122753 (built once per
    session).  For e4m3 the lm_head is quantised by the library's host quantiser after a slice of it
    has been checked bit for bit against the oracle's (the numpy quantiser needs a minute for it)."""
    import stack_util as su
    if "w" not in _FULL:
        _FULL["w"] = su.make_weights(2, 2304, 3456, 5760, 122753, seed=7700)
    w = _FULL["w"]
    if fp8 and "q" not in _FULL:
        q = {"layers": []}
        for lay in w["layers"]:
            q["layers"].append({k: onp.make_fp8_weight(lay[k]) for k in ("qkv", "o", "gate_up", "down")})
        lm = w["lm_head"]
        got_q, got_s = pkg.quantize_rows_host(lm)
        ref_q, ref_s = onp.make_fp8_weight(lm[:4096])
        assert np.array_equal(got_q[:4096], ref_q) and np.array_equal(got_s[:4096], ref_s)
        q["lm_head"] = (got_q, got_s)
        _FULL["q"] = q
    return w, _FULL.get("q")


def _oracle_full(w, q, x, fp8):
    H = w["final_norm"].size

    def lin(mat, qs, v):
        return onp.linear_fp8(qs[0], qs[1], v) if fp8 else onp.linear_bf16(mat, v)

    res = x.copy()
    for l, lay in enumerate(w["layers"]):
        ql = q["layers"][l] if fp8 else {k: None for k in ("qkv", "o", "gate_up", "down")}
        h = onp.rmsnorm_bf16(lay["norm1"], res)
        qkv = lin(lay["qkv"], ql["qkv"], h)
        res = onp.add_bf16(res, lin(lay["o"], ql["o"], np.ascontiguousarray(qkv[..., :H])))
        h = onp.rmsnorm_bf16(lay["norm2"], res)
        gu = lin(lay["gate_up"], ql["gate_up"], h)
        I = gu.shape[-1] // 2
        res = onp.add_bf16(res, lin(lay["down"], ql["down"], onp.swiglu_bf16(gu[..., :I], gu[..., I:])))
    return lin(w["lm_head"], q["lm_head"] if fp8 else None, onp.rmsnorm_bf16(w["final_norm"], res))


def _upload_full(pkg, torch, desc, w, q, fp8):
    wbytes, sbytes = pkg.stack_sizes(desc)
    arena = torch.zeros(wbytes, dtype=torch.uint8, device="cuda")
    scratch = torch.zeros(sbytes, dtype=torch.uint8, device="cuda")

    def put(layer, name, arr):
        off, n = pkg.stack_section(desc, layer, name)
        b = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        assert b.size == n, (name, b.size, n)
        arena[off:off + n] = torch.from_numpy(b).cuda()

    def il(a):
        I = a.shape[0] // 2
        out = np.empty_like(a)
        out[0::2], out[1::2] = a[:I], a[I:]
        return out

    for l, lay in enumerate(w["layers"]):
        for name in ("qkv", "o", "gate_up", "down"):
            f = il if name == "gate_up" else (lambda a: a)
            if fp8:
                put(l, name, f(q["layers"][l][name][0])); put(l, name + "_scale", f(q["layers"][l][name][1]))
            else:
                put(l, name, f(lay[name]))
        put(l, "norm1", lay["norm1"]); put(l, "norm2", lay["norm2"])
    if fp8:
        put(0, "lm_head", q["lm_head"][0]); put(0, "lm_head_scale", q["lm_head"][1])
    else:
        put(0, "lm_head", w["lm_head"])
    put(0, "final_norm", w["final_norm"])
    return arena, scratch


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("M", [1, 8])
def test_stack_at_benchmark_dimensions(pkg, fp8, M):
    """hidden 2304, qkv 3456, inter 5760, vocab 122753 -- the shapes the benchmark streams -- against
    the oracle chain: every kernel choice the 40-layer run makes (tile shapes, rounds, ragged vocab,
    L2 prefetch hints from one linear to the next) is exercised here with two layers."""
    torch = pytest.importorskip("torch")
    layers, H, Q, I, V = 2, 2304, 3456, 5760, 122753
    w, q = _full_weights(pkg, fp8)
    desc = pkg.stack_desc(layers, H, Q, I, V, fp8=fp8, max_batch=8)
    arena, scratch = _upload_full(pkg, torch, desc, w, q, fp8)
    st = pkg.stack_create(desc, arena, scratch)
    try:
        x = onp.seeded_bf16(7800 + M, (M, H), 1.0)
        hx = torch.from_numpy(x.view(np.int16)).pin_memory()
        htok = torch.full((M,), -1, dtype=torch.int32).pin_memory()
        stream = torch.cuda.Stream()
        toks = []
        for _ in range(3):                          # eager, replay, replay: identical tokens
            pkg.stack_step_host(st, hx, M, htok, stream)
            toks.append(htok.clone())
        assert all(torch.equal(toks[0], t) for t in toks[1:])
        assert pkg.stack_exchange_status(st, stream) == 0
        ref = _oracle_full(w, q, x if M > 1 else x[0], fp8).reshape(M, V)
        off = pkg.stack_logits_ptr(st) - scratch.data_ptr()
        got = scratch[off:off + M * V * 2].cpu().numpy().view(np.uint16).reshape(M, V)
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
        # the L2 prefetch (off by default) changes where the weights come from, never the result
        pkg.debug_set_prefetch(mode=1)
        try:
            pkg.stack_step(st, torch.from_numpy(x.view(np.int16)).cuda(), M, torch.zeros(M, dtype=torch.int32, device="cuda"))
            torch.cuda.synchronize()
            again = scratch[off:off + M * V * 2].cpu().numpy().view(np.uint16).reshape(M, V)
            assert np.array_equal(again, got)
        finally:
            pkg.debug_set_prefetch(mode=0)
        if M == 1:
            # the one-launch form of the M = 1 step (off by default): same bits, same token, three steps in a row
            # (its arrival counters and tags carry over from step to step), no wait ran out
            pkg.debug_set_chain(True)
            try:
                dx = torch.from_numpy(x.view(np.int16)).cuda()
                dtok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
                for _ in range(3):
                    scratch[off:off + V * 2].zero_()
                    pkg.stack_step(st, dx, 1, dtok)
                    torch.cuda.synchronize()
                    chain = scratch[off:off + V * 2].cpu().numpy().view(np.uint16).reshape(1, V)
                    assert np.array_equal(chain, got)
                    assert int(dtok.item()) == int(toks[0][0])
                assert pkg.stack_exchange_status(st, stream) == 0
            finally:
                pkg.debug_set_chain(False)
    finally:
        pkg.stack_destroy(st)
