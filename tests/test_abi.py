"""CPU: the C-ABI library loads and exports every symbol the header declares,
and the ctypes signature table covers the header one to one (no compute calls)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for h in ("mc_sm100a_linear.h", "mc_sm100a_runtime.h"):
        txt = open(os.path.join(ROOT, "include", h)).read()
        names |= set(re.findall(r"MC_SM100_API[^;(]*?\b(mc_sm100_\w+)\s*\(", txt))
    return sorted(names)


def test_header_declares_entry_points():
    names = _declared()
    assert len(names) >= 20
    for must in ("mc_sm100_decode_gemv", "mc_sm100_gemv_fp8", "mc_sm100_gemv_fp8_rows_m", "mc_sm100_gemm_bf16",
                 "mc_sm100_gate_up_swiglu", "mc_sm100_lm_head_argmax", "mc_sm100_last_error", "mc_sm100_model_load",
                 "mc_sm100_decode_one", "mc_sm100_batch_group_create", "mc_sm100_batch_step"):
        assert must in names


def test_library_exports_every_declared_symbol(pkg):
    assert os.path.exists(pkg.LIB_PATH), "build the library first (python minicpm5-5080fast_b200/build.py)"
    h = ctypes.CDLL(pkg.LIB_PATH)
    for name in _declared():
        assert hasattr(h, name), f"{name} is declared in the header but not exported"


def test_ctypes_table_matches_header(pkg):
    assert sorted(pkg.SIGNATURES) == _declared()


def test_status_codes_match_reference_values():
    txt = open(os.path.join(ROOT, "include", "mc_sm100a_linear.h")).read()
    want = {"MC_OK": 0, "MC_E_INVALID_ARGUMENT": 1, "MC_E_IO": 2, "MC_E_CUDA": 3, "MC_E_MODEL_MISMATCH": 4,
            "MC_E_OUT_OF_MEMORY": 5, "MC_E_GRAPH": 6, "MC_E_UNSUPPORTED": 7, "MC_E_INTERNAL": 100}
    for k, v in want.items():
        assert re.search(rf"\b{k} = {v}\b", txt), k


def test_argument_validation_needs_no_gpu(pkg):
    """Bad arguments are rejected before any CUDA call, with a message."""
    lib = pkg.lib()
    assert lib.mc_sm100_decode_gemv(None, None, None, 8, 8, 1, 0, None, None, 0) == pkg.MC_E_INVALID_ARGUMENT
    assert "invalid args" in pkg.last_error()
    assert lib.mc_sm100_gemv_fp8(None, None, None, None, 0, 0, None, 0) == pkg.MC_E_INVALID_ARGUMENT
    assert lib.mc_sm100_gemv_fp8_rows_m(1, 1, 1, 1, 65, 8, 16, None, 0) == pkg.MC_E_INVALID_ARGUMENT
    assert "M=65" in pkg.last_error()
    # tactic 0 (library GEMM) does not exist here
    assert lib.mc_sm100_decode_gemv(16, 16, 16, 8, 8, 0, 0, None, None, 0) == pkg.MC_E_INVALID_ARGUMENT
    assert "tactic" in pkg.last_error()
    # split-K: K/S must be a multiple of 8 and a partial buffer is required
    assert lib.mc_sm100_decode_gemv(16, 16, 16, 8, 24, 2, 2, 16, None, 0) == pkg.MC_E_INVALID_ARGUMENT
    assert lib.mc_sm100_decode_gemv(16, 16, 16, 8, 32, 2, 2, None, None, 0) == pkg.MC_E_INVALID_ARGUMENT
    assert lib.mc_sm100_argmax_stage_bytes(1) >= 8 * 1024


def test_shared_memory_opt_in_bookkeeping_is_per_device(pkg):
    """A process that drives several GPUs must raise a kernel's dynamic shared memory once on EVERY device (the
    attribute is per device), remember it per device and size, and survive racing host threads: the library's
    host-only self-test of that bookkeeping (no CUDA call, no GPU needed)."""
    assert pkg.lib().mc_sm100_debug_optin_selftest() == 0
