"""Synthetic decode stack shared by the stack tests: numpy weights in the packed-file
order (gate | up row-concatenated), the oracle chain, and the arena upload."""
import numpy as np

import oracle_np as onp


def make_weights(layers, H, Q, I, V, seed=500):
    w = {"layers": []}
    for l in range(layers):
        w["layers"].append({
            "qkv": onp.seeded_bf16(seed + 10 * l + 0, (Q, H), 0.02), "o": onp.seeded_bf16(seed + 10 * l + 1, (H, H), 0.02),
            "gate_up": onp.seeded_bf16(seed + 10 * l + 2, (2 * I, H), 0.02), "down": onp.seeded_bf16(seed + 10 * l + 3, (H, I), 0.02),
            "norm1": onp.f32_to_bf16(1.0 + 0.1 * np.random.default_rng(seed + 10 * l + 4).standard_normal(H).astype(np.float32)),
            "norm2": onp.f32_to_bf16(1.0 + 0.1 * np.random.default_rng(seed + 10 * l + 5).standard_normal(H).astype(np.float32))})
    w["lm_head"] = onp.seeded_bf16(seed + 9000, (V, H), 0.02)
    w["final_norm"] = onp.f32_to_bf16(1.0 + 0.1 * np.random.default_rng(seed + 9001).standard_normal(H).astype(np.float32))
    return w


def oracle_stack(w, x, fp8):
    """Per layer: h = rmsnorm1(x); qkv = Wqkv h; x += Wo qkv[:H]; h = rmsnorm2(x); x += Wd swiglu(Wgu h);
    then logits = Wlm rmsnorm_f(x).  Every intermediate is bf16, as the device stores it."""
    H = w["final_norm"].size

    def lin(mat, v):
        if fp8:
            q, sc = onp.make_fp8_weight(mat)
            return onp.linear_fp8(q, sc, v)
        return onp.linear_bf16(mat, v)

    res = x.copy()
    for lay in w["layers"]:
        h = onp.rmsnorm_bf16(lay["norm1"], res)
        qkv = lin(lay["qkv"], h)
        res = onp.add_bf16(res, lin(lay["o"], np.ascontiguousarray(qkv[..., :H])))
        h = onp.rmsnorm_bf16(lay["norm2"], res)
        gu = lin(lay["gate_up"], h)
        I = gu.shape[-1] // 2
        res = onp.add_bf16(res, lin(lay["down"], onp.swiglu_bf16(gu[..., :I], gu[..., I:])))
    logits = lin(w["lm_head"], onp.rmsnorm_bf16(w["final_norm"], res))
    return logits


def upload(pkg, torch, desc, w, fp8):
    """Fills a device weight arena at the library's section offsets: gate_up (and its
    scales) interleaved (gate_j, up_j), every other section as packed."""
    wbytes, sbytes = pkg.stack_sizes(desc)
    arena = torch.zeros(wbytes, dtype=torch.uint8, device="cuda")
    scratch = torch.zeros(sbytes, dtype=torch.uint8, device="cuda")

    def put(layer, name, arr):
        off, n = pkg.stack_section(desc, layer, name)
        b = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        assert b.size == n, (name, b.size, n)
        arena[off:off + n] = torch.from_numpy(b).cuda()

    def interleave(a):
        I = a.shape[0] // 2
        out = np.empty_like(a)
        out[0::2], out[1::2] = a[:I], a[I:]
        return out

    def put_mat(layer, name, mat, il=False):
        if fp8:
            q, sc = onp.make_fp8_weight(mat)
            put(layer, name, interleave(q) if il else q)
            put(layer, name + "_scale", interleave(sc) if il else sc)
        else:
            put(layer, name, interleave(mat) if il else mat)

    for l, lay in enumerate(w["layers"]):
        put_mat(l, "qkv", lay["qkv"]); put_mat(l, "o", lay["o"]); put_mat(l, "gate_up", lay["gate_up"], il=True)
        put_mat(l, "down", lay["down"]); put(l, "norm1", lay["norm1"]); put(l, "norm2", lay["norm2"])
    put_mat(0, "lm_head", w["lm_head"]); put(0, "final_norm", w["final_norm"])
    return arena, scratch
