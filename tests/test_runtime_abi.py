"""The model / session / batch-group entry points (include/mc_sm100a_runtime.h): a C++ host on a
synthetic model, and a packed weight file loaded from disk whose tokens and logits are checked
against the oracle chain."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import oracle_np as onp
import wpk_np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "runtime_smoke.cpp")
LIBDIR = os.path.join(ROOT, "minicpm5-5080fast_b200")


def _build(tmp_path):
    exe = str(tmp_path / "runtime_smoke")
    cmd = ["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe, "-L", LIBDIR, "-lmc_sm100a_linear",
           "-Wl,-rpath," + LIBDIR]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_runtime_header_compiles_and_validates_without_a_gpu(pkg, tmp_path):
    """CPU: the header is plain C for a host compiler, every entry point links, and the argument checks that
    come before any device use answer as the reference's do (the run stops at the first call that needs a GPU)."""
    exe = _build(tmp_path)
    out = subprocess.run([exe, str(tmp_path / "model_dir")], capture_output=True, text=True, timeout=60)
    import torch
    if not torch.cuda.is_available():
        # every REQUIRE before the first successful load passed; the load itself needs the device
        assert "FAILED line" in out.stdout and "mc_sm100_model_load(dir, &o, &m) == MC_OK" in out.stdout, out.stdout


@pytest.mark.gpu
def test_runtime_smoke_runs(pkg, tmp_path):
    exe = _build(tmp_path)
    out = subprocess.run([exe, str(tmp_path / "model_dir")], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "RUNTIME-SMOKE-OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def _write_model(tmp_path, fp8, layers=2, H=256, Q=384, I=512, V=1500, seed=4100):
    import stack_util as su
    w = su.make_weights(layers, H, Q, I, V, seed=seed)
    emb = onp.seeded_bf16(seed + 9500, (V, H), 1.0)

    def mat(name, a):
        if fp8:
            q, sc = onp.make_fp8_weight(a)
            return (name, q, sc)
        return (name, a)

    secs = [("embedding", emb), mat("lm_head", w["lm_head"]), ("final_norm", w["final_norm"])]
    for l, lay in enumerate(w["layers"]):
        secs += [(f"layer{l}.norm1", lay["norm1"]), mat(f"layer{l}.qkv", lay["qkv"]), mat(f"layer{l}.o", lay["o"]),
                 (f"layer{l}.norm2", lay["norm2"]), mat(f"layer{l}.gate_up", lay["gate_up"]), mat(f"layer{l}.down", lay["down"])]
    d = tmp_path / ("model_fp8" if fp8 else "model_bf16")
    d.mkdir()
    wpk_np.write_wpk(str(d / "model.wpk"), secs)
    return str(d), w, emb


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_packed_file_to_tokens_matches_oracle(pkg, tmp_path, fp8):
    """model.wpk (the reference's container, gate|up row-concatenated as its packer writes them) -> mc_sm100_model_load
    -> prefill / decode_one: every step's logits within tolerance of the oracle chain on the embedded token, tokens
    equal to the oracle's greedy choice whenever its two best logits are clearly apart, batch steps likewise."""
    import stack_util as su
    model_dir, w, emb = _write_model(tmp_path, fp8)
    V, H = emb.shape
    m = pkg.model_load(model_dir, pkg.model_options(fp8=fp8, max_sessions=8))
    try:
        assert pkg.model_dims(m) == (2, 256, 384, 512, 1500)
        with pytest.raises(pkg.McError) as e:                 # the file's matrices are not of the precision asked for
            pkg.model_load(model_dir, pkg.model_options(fp8=not fp8))
        assert e.value.status == 4
        s = pkg.session_create(m)
        cfg = pkg.greedy_config()
        pkg.prefill(s, [7, 8, 9])
        tok_in = 9
        for step in range(5):
            ref = su.oracle_stack(w, emb[tok_in], fp8)
            got = pkg.session_logits(s, V)
            gf, rf = onp.bf16_to_f32(got).astype(np.float64), onp.bf16_to_f32(ref).astype(np.float64)
            assert np.sqrt(((gf - rf) ** 2).sum() / (rf ** 2).sum()) < 1e-2
            want = onp.greedy(got)
            top = np.sort(rf)[-2:]
            if top[1] - top[0] > 0.05:
                assert want == int(np.argmax(rf))
            tok = pkg.decode_one(s, cfg)                      # hands out the decision taken on tok_in ...
            assert tok == want
            tok_in = tok                                      # ... and has already run the step on it
        st = pkg.get_stats(s)
        assert st.prompt_tokens == 3 and st.generated_tokens == 5
        # three members in a group: each row's hand-out equals what its solo session decided
        ss = [pkg.session_create(m) for _ in range(3)]
        expect = []
        for i, t in enumerate(ss):
            pkg.prefill(t, [100 + i])
            expect.append(onp.greedy(pkg.session_logits(t, V)))
        g = pkg.batch_group_create(m, 8)
        slots = [pkg.batch_group_add(g, t) for t in ss]
        assert slots == [0, 1, 2]
        out = pkg.batch_step(g, slots, [cfg] * 3)
        assert out == expect
        out2 = pkg.batch_step(g, slots, [cfg] * 3)            # decisions of the batched step on those tokens
        for i in range(3):
            ref = onp.bf16_to_f32(su.oracle_stack(w, emb[out[i]], fp8)).astype(np.float64)
            top = np.sort(ref)[-2:]
            if top[1] - top[0] > 0.05:
                assert out2[i] == int(np.argmax(ref))
        assert pkg.batch_group_stats(g)["steps"] == 2
        pkg.batch_group_destroy(g)
        for t in ss + [s]:
            pkg.session_destroy(t)
    finally:
        pkg.model_destroy(m)
