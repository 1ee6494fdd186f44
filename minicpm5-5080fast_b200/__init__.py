"""ctypes view of libmc_sm100a_linear.so -- the B200 decode linear-layer library.

The product is the C-ABI shared library (`include/mc_sm100a_linear.h`); this
module only loads it and gives tests and the benchmark functions with the
reference launchers' names and argument order
(native/kernels/sm120/kernels.h:657-798, native/runtime/gemm.h:39-90).
PyTorch tensors are used purely as device-memory handles (`data_ptr()`); there
is no PyTorch, Triton or CPU implementation behind any call: if the library is
missing or a call fails, an exception is raised.

The directory name contains a hyphen, so import it with
`importlib.import_module("minicpm5-5080fast_b200")`.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmc_sm100a_linear.so")

MC_OK = 0
MC_E_INVALID_ARGUMENT = 1
MC_E_CUDA = 3
MC_E_UNSUPPORTED = 7
TACTIC_ROWS, TACTIC_SPLITK, TACTIC_FP8 = 1, 2, 3

_u16p = C.c_void_p
_vp = C.c_void_p
_u32 = C.c_uint32
_i32 = C.c_int32

# name -> (restype, argtypes): mirrors include/mc_sm100a_linear.h one to one
SIGNATURES = {
    "mc_sm100_last_error": (C.c_char_p, []),
    "mc_sm100_device_check": (_i32, [C.POINTER(_i32), C.POINTER(C.c_uint64), C.POINTER(_i32), C.POINTER(_i32)]),
    "mc_sm100_decode_gemv": (_i32, [_vp, _vp, _vp, _u32, _u32, _i32, _u32, _vp, _vp, _i32]),
    "mc_sm100_decode_gemv_splitk_static": (_i32, [_vp, _vp, _vp, _u32, _u32, _u32, _vp, _i32]),
    "mc_sm100_gemv_fp8": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, _vp, _i32]),
    "mc_sm100_gemv_rows_prologue": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_float, _vp, _i32]),
    "mc_sm100_gemv_fp8_prologue": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_float, _vp, _i32]),
    "mc_sm100_gemv_rows_swiglu": (_i32, [_vp, _vp, _vp, _u32, _u32, _vp, _i32]),
    "mc_sm100_gemv_fp8_swiglu": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, _vp, _i32]),
    "mc_sm100_gate_up_swiglu": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp, _i32]),
    "mc_sm100_gate_up_swiglu_prologue": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_float, _vp, _i32]),
    "mc_sm100_interleave_rows": (_i32, [_vp, _vp, _u32, _u32, _vp]),
    "mc_sm100_gemv_fp8_rows_m": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp, _i32]),
    "mc_sm100_gemm_bf16": (_i32, [_vp, _vp, C.c_size_t, _u32, _u32, _u32, _vp, _vp, _vp]),
    "mc_sm100_gemm_workspace_bytes": (C.c_size_t, [_u32, _u32, _u32]),
    "mc_sm100_gemm_fp8_q": (_i32, [_vp, _vp, C.c_size_t, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp]),
    "mc_sm100_gemm_fp8": (_i32, [_vp, _vp, C.c_size_t, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mc_sm100_quant_rows": (_i32, [_vp, _vp, _vp, _u32, _u32, _vp]),
    "mc_sm100_post_scale_rows": (_i32, [_vp, _vp, _vp, _u32, _u32, _vp]),
    "mc_sm100_residual_rmsnorm_rows": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, C.c_float, _vp, _i32]),
    "mc_sm100_argmax_bf16": (_i32, [_vp, _u32, _u32, _u32, _i32, _vp, _vp, _vp, _vp, _i32]),
    "mc_sm100_argmax_stage_bytes": (C.c_size_t, [_u32]),
    "mc_sm100_lm_head_argmax": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _i32, _vp, _vp, _vp, _vp, _i32]),
    "mc_sm100_lm_head_argmax_prologue": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_float, _i32,
                                                _vp, _vp, _vp, _vp, _i32]),
    "mc_sm100_gemv_pick_split_s": (_u32, [_u32, _u32]),
    "mc_sm100_gemv_partial_floats": (C.c_size_t, [_u32]),
    "mc_sm100_select_decode_gemv_tactic": (_i32, [_vp, _u32, _u32, _vp, _vp, _vp, C.c_size_t, _vp, C.c_size_t, _vp, _vp]),
    "mc_sm100_run_decode_gemv": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, _vp, _vp, _i32]),
    "mc_sm100_sample_topk_topp": (_i32, [_vp, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _i32]),
    "mc_sm100_sampling_exchange_bytes": (C.c_size_t, [_u32, _u32]),
    "mc_sm100_sample_topk_topp_sharded": (_i32, [_vp, _u32, _u32, _u32, _i32, _vp, _vp, _vp, _vp, _vp, _u32, _vp, _u32, _u32,
                                                 C.c_uint64, _vp, _vp, _i32]),
    "mc_sm100_linear_host": (_i32, [_i32, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp, C.c_size_t, _vp]),
    "mc_sm100_stack_sizes": (_i32, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "mc_sm100_stack_section": (_i32, [_vp, _u32, _u32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "mc_sm100_stack_create": (_i32, [_vp, _vp, _vp, C.POINTER(_vp)]),
    "mc_sm100_stack_destroy": (None, [_vp]),
    "mc_sm100_stack_logits": (_vp, [_vp]),
    "mc_sm100_stack_status_word": (_vp, [_vp]),
    "mc_sm100_stack_step": (_i32, [_vp, _vp, _u32, _vp, _vp]),
    "mc_sm100_stack_step_host": (_i32, [_vp, _vp, _u32, _vp, _vp]),
    "mc_sm100_stack_exchange_bytes": (_i32, [_vp, C.POINTER(C.c_uint64)]),
    "mc_sm100_stack_bind_exchange": (_i32, [_vp, _vp, C.c_uint64, _vp]),
    "mc_sm100_stack_exchange_status": (_i32, [_vp, C.POINTER(_i32), _vp]),
    "mc_sm100_gemv_sharded": (_i32, [_i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_float, _vp, _vp, _i32]),
    "mc_sm100_lm_head_argmax_sharded": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_float, _i32,
                                               _vp, _vp, _vp, _vp, _vp, _i32]),
    "mc_sm100_peer_argmax": (_i32, [_vp, _vp, _u32, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_uint64, _vp, _vp, _vp, _vp, _i32]),
    "mc_sm100_peer_allgather_rows": (_i32, [_vp, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _u32, _u32, C.c_uint64, _vp, _vp, _i32]),
    "mc_sm100_peer_allgather": (_i32, [_vp, _u32, _u32, _vp, _vp, _vp, _vp, _u32, _u32, C.c_uint64, _vp, _vp, _i32]),
    "mc_sm100_wpk_name_hash": (C.c_uint64, [C.c_char_p]),
    "mc_sm100_wpk_open": (_i32, [C.c_char_p, C.POINTER(_vp)]),
    "mc_sm100_wpk_close": (None, [_vp]),
    "mc_sm100_wpk_section_count": (_u32, [_vp]),
    "mc_sm100_wpk_find": (_i32, [_vp, C.c_char_p, _vp]),
    "mc_sm100_wpk_upload": (_i32, [_vp, C.c_char_p, _u32, _u32, _i32, _vp, C.c_uint64, _vp, _vp]),
    "mc_sm100_wpk_writer_create": (_i32, [C.c_char_p, _u32, _u32, _vp, C.POINTER(_vp)]),
    "mc_sm100_wpk_writer_add": (_i32, [_vp, C.c_char_p, _u32, _u32, _vp, _vp, _vp]),
    "mc_sm100_wpk_writer_finish": (_i32, [_vp]),
    "mc_sm100_wpk_writer_abort": (None, [_vp]),
    "mc_sm100_quantize_rows_host": (_i32, [_vp, _u32, _u32, _vp, _vp]),
    "mc_sm100_e4m3_from_f32_host": (_i32, [_vp, C.c_uint64, _vp]),
    # include/mc_sm100a_runtime.h (handles are 8-byte structs passed by value: one pointer)
    "mc_sm100_model_load": (_i32, [C.c_char_p, _vp, C.POINTER(_vp)]),
    "mc_sm100_model_destroy": (None, [_vp]),
    "mc_sm100_session_create": (_i32, [_vp, C.POINTER(_vp)]),
    "mc_sm100_session_reset": (_i32, [_vp]),
    "mc_sm100_session_destroy": (None, [_vp]),
    "mc_sm100_prefill": (_i32, [_vp, _vp, _u32]),
    "mc_sm100_decode_one": (_i32, [_vp, _vp, C.POINTER(_i32)]),
    "mc_sm100_get_stats": (_i32, [_vp, _vp]),
    "mc_sm100_batch_group_create": (_i32, [_vp, _vp, C.POINTER(_vp)]),
    "mc_sm100_batch_group_add": (_i32, [_vp, _vp, C.POINTER(_u32)]),
    "mc_sm100_batch_group_remove": (_i32, [_vp, _u32]),
    "mc_sm100_batch_step": (_i32, [_vp, _vp, _u32, _vp, _vp]),
    "mc_sm100_batch_group_destroy": (None, [_vp]),
    "mc_sm100_debug_batch_group_stats": (_i32, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(_u32), C.POINTER(_u32)]),
    "mc_sm100_debug_model_dims": (_i32, [_vp, C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32)]),
    "mc_sm100_debug_session_logits": (_i32, [_vp, _vp, _u32]),
    "mc_sm100_hint_next_weights": (None, [_vp, C.c_uint64]),
    "mc_sm100_debug_set_prefetch": (None, [_i32, _i32, _i32, C.c_int64]),
    "mc_sm100_debug_set_chain": (None, [_i32]),
    "mc_sm100_debug_optin_selftest": (_i32, []),
    "mc_sm100_debug_set_mma_rows": (None, [_i32]),
    "mc_sm100_debug_mma_rows_plan": (None, [_u32, _u32, _vp, _vp, _vp]),
    "mc_sm100_debug_chain_plan": (None, [_i32, _u32, _u32, _vp, _vp, _vp, _vp]),
    "mc_sm100_debug_set_math": (None, [_i32, _i32]),
    "mc_sm100_debug_take_error": (_i32, []),
}


class McError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"mc_status {status}: {message}")
        self.status = status
        self.message = message


_lib = None


def lib() -> C.CDLL:
    """Loads the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python minicpm5-5080fast_b200/build.py`; "
                "there is no fallback implementation")
        h = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


def last_error() -> str:
    return (lib().mc_sm100_last_error() or b"").decode()


def _check(status: int) -> None:
    if status != MC_OK:
        raise McError(status, last_error())


def _p(t) -> int | None:
    """Device (or pinned host) address of a tensor, None passes NULL."""
    if t is None:
        return None
    return int(t) if isinstance(t, int) else t.data_ptr()


def _stream(stream) -> int | None:
    if stream is None:
        import torch
        stream = torch.cuda.current_stream()
    s = stream if isinstance(stream, int) else stream.cuda_stream
    return s or None


# ---- launchers, named after the reference's ------------------------------------------
def device_check():
    sm, l2, mj, mn = _i32(), C.c_uint64(), _i32(), _i32()
    _check(lib().mc_sm100_device_check(C.byref(sm), C.byref(l2), C.byref(mj), C.byref(mn)))
    return {"sm_count": sm.value, "l2_bytes": l2.value, "cc": (mj.value, mn.value)}


def launch_decode_gemv(w, x, y, N, K, tactic=TACTIC_ROWS, split_s=0, split_partial=None, stream=None, pdl=False):
    _check(lib().mc_sm100_decode_gemv(_p(w), _p(x), _p(y), N, K, tactic, split_s, _p(split_partial),
                                      _stream(stream), int(pdl)))


def launch_decode_gemv_splitk_static(w, x, y, N, K, split_s, stream=None, pdl=False):
    _check(lib().mc_sm100_decode_gemv_splitk_static(_p(w), _p(x), _p(y), N, K, split_s, _stream(stream), int(pdl)))


def launch_gemv_fp8(w, scale, x, y, N, K, stream=None, pdl=False):
    _check(lib().mc_sm100_gemv_fp8(_p(w), _p(scale), _p(x), _p(y), N, K, _stream(stream), int(pdl)))


def launch_gemv_rows_prologue(w, res_in, addend, norm_w, res_out, y, N, n, eps, stream=None, pdl=False):
    _check(lib().mc_sm100_gemv_rows_prologue(_p(w), _p(res_in), _p(addend), _p(norm_w), _p(res_out), _p(y),
                                             N, n, eps, _stream(stream), int(pdl)))


def launch_gemv_fp8_prologue(w, scale, res_in, addend, norm_w, res_out, y, N, n, eps, stream=None, pdl=False):
    _check(lib().mc_sm100_gemv_fp8_prologue(_p(w), _p(scale), _p(res_in), _p(addend), _p(norm_w), _p(res_out),
                                            _p(y), N, n, eps, _stream(stream), int(pdl)))


def launch_gemv_rows_swiglu(w, gate_up, y, N, K, stream=None, pdl=False):
    _check(lib().mc_sm100_gemv_rows_swiglu(_p(w), _p(gate_up), _p(y), N, K, _stream(stream), int(pdl)))


def launch_gemv_fp8_swiglu(w, scale, gate_up, y, N, K, stream=None, pdl=False):
    _check(lib().mc_sm100_gemv_fp8_swiglu(_p(w), _p(scale), _p(gate_up), _p(y), N, K, _stream(stream), int(pdl)))


def launch_gate_up_swiglu(w_il, scale_il, x, y, M, N, K, stream=None, pdl=False):
    _check(lib().mc_sm100_gate_up_swiglu(_p(w_il), _p(scale_il), _p(x), _p(y), M, N, K, _stream(stream), int(pdl)))


def launch_gate_up_swiglu_prologue(w_il, scale_il, res_in, addend, norm_w, res_out, y, N, n, eps,
                                   stream=None, pdl=False):
    _check(lib().mc_sm100_gate_up_swiglu_prologue(_p(w_il), _p(scale_il), _p(res_in), _p(addend), _p(norm_w),
                                                  _p(res_out), _p(y), N, n, eps, _stream(stream), int(pdl)))


def interleave_rows(src, dst, I, row_bytes, stream=None):
    _check(lib().mc_sm100_interleave_rows(_p(src), _p(dst), I, row_bytes, _stream(stream)))


def launch_gemv_fp8_rows_m(w, scale, x, y, M, N, K, stream=None, pdl=False):
    _check(lib().mc_sm100_gemv_fp8_rows_m(_p(w), _p(scale), _p(x), _p(y), M, N, K, _stream(stream), int(pdl)))


def gemm_workspace_bytes(M, N, K) -> int:
    return lib().mc_sm100_gemm_workspace_bytes(M, N, K)


def gemm_bf16(stream, workspace, ws_size, M, N, K, a_weight, b_act, c):
    _check(lib().mc_sm100_gemm_bf16(_stream(stream), _p(workspace), ws_size, M, N, K, _p(a_weight), _p(b_act), _p(c)))


def gemm_fp8_q(stream, workspace, ws_size, M, N, K, w_fp8, w_scale, x_fp8, x_scale, y):
    _check(lib().mc_sm100_gemm_fp8_q(_stream(stream), _p(workspace), ws_size, M, N, K, _p(w_fp8), _p(w_scale),
                                     _p(x_fp8), _p(x_scale), _p(y)))


def gemm_fp8(stream, workspace, ws_size, M, N, K, w_fp8, w_scale, x_bf16, y, x_fp8_scratch, x_scale_scratch):
    _check(lib().mc_sm100_gemm_fp8(_stream(stream), _p(workspace), ws_size, M, N, K, _p(w_fp8), _p(w_scale),
                                   _p(x_bf16), _p(y), _p(x_fp8_scratch), _p(x_scale_scratch)))


def launch_quant_rows(x, xq, scale, M, K, stream=None):
    _check(lib().mc_sm100_quant_rows(_p(x), _p(xq), _p(scale), M, K, _stream(stream)))


def launch_post_scale_rows(y, w_scale, x_scale, M, N, stream=None):
    _check(lib().mc_sm100_post_scale_rows(_p(y), _p(w_scale), _p(x_scale), M, N, _stream(stream)))


def launch_residual_rmsnorm_rows(res, add, norm_w, out, rows, n, eps, stream=None, pdl=False):
    _check(lib().mc_sm100_residual_rmsnorm_rows(_p(res), _p(add), _p(norm_w), _p(out), rows, n, eps, _stream(stream), int(pdl)))


def argmax_stage_bytes(n_rows) -> int:
    return lib().mc_sm100_argmax_stage_bytes(n_rows)


def launch_argmax_bf16(logits, n_rows, vocab, row_stride, index_base, stage, out_idx, out_val=None,
                       stream=None, pdl=False):
    _check(lib().mc_sm100_argmax_bf16(_p(logits), n_rows, vocab, row_stride, index_base, _p(stage), _p(out_idx),
                                      _p(out_val), _stream(stream), int(pdl)))


def launch_lm_head_argmax(w, scale, x, logits, y_stride, M, N, K, index_base, stage, out_idx, out_val=None,
                          stream=None, pdl=False):
    _check(lib().mc_sm100_lm_head_argmax(_p(w), _p(scale), _p(x), _p(logits), y_stride, M, N, K, index_base,
                                         _p(stage), _p(out_idx), _p(out_val), _stream(stream), int(pdl)))


def launch_lm_head_argmax_prologue(w, scale, res_in, addend, norm_w, res_out, logits, N, n, eps, index_base,
                                   stage, out_idx, out_val=None, stream=None, pdl=False):
    _check(lib().mc_sm100_lm_head_argmax_prologue(_p(w), _p(scale), _p(res_in), _p(addend), _p(norm_w),
                                                  _p(res_out), _p(logits), N, n, eps, index_base, _p(stage),
                                                  _p(out_idx), _p(out_val), _stream(stream), int(pdl)))


class GemvTactic(C.Structure):
    _fields_ = [("struct_size", _u32), ("tactic", _i32), ("split_s", _u32), ("best_split_s", _u32), ("us_rows", C.c_float),
                ("us_splitk", C.c_float), ("reserved", _u32 * 2)]


def select_decode_gemv_tactic(w, N, K, x, y, partial=None, partial_floats=0, flush=None, stream=None) -> GemvTactic:
    t = GemvTactic()
    _check(lib().mc_sm100_select_decode_gemv_tactic(_p(w), N, K, _p(x), _p(y), _p(partial), partial_floats, _p(flush),
                                                    flush.numel() * flush.element_size() if flush is not None else 0,
                                                    _stream(stream), C.cast(C.byref(t), _vp)))
    return t


def run_decode_gemv(tactic, w, x, y, N, K, partial=None, stream=None, pdl=False):
    _check(lib().mc_sm100_run_decode_gemv(C.cast(C.byref(tactic), _vp), _p(w), _p(x), _p(y), N, K, _p(partial), _stream(stream), int(pdl)))


def sample_topk_topp(logits, n_rows, vocab, row_stride, cfg, rng_state, out_token, stream=None, pdl=False):
    """cfg: device tensor of n_rows x 6 words (temperature, top_p as f32 bits, top_k, rep_penalty, 0, 0)."""
    _check(lib().mc_sm100_sample_topk_topp(_p(logits), n_rows, vocab, row_stride, _p(cfg), _p(rng_state), _p(out_token),
                                           _stream(stream), int(pdl)))


def sampling_exchange_bytes(max_rows, world) -> int:
    return lib().mc_sm100_sampling_exchange_bytes(max_rows, world)


def sample_topk_topp_sharded(logits, n_rows, vocab, row_stride, index_base, cfg, rng_state, out_token, region_peers, my_region,
                             max_rows, step, rank, world, status, timeout_ns=0, stream=None, pdl=False):
    _check(lib().mc_sm100_sample_topk_topp_sharded(_p(logits), n_rows, vocab, row_stride, index_base, _p(cfg), _p(rng_state),
                                                   _p(out_token), _p(region_peers), _p(my_region), max_rows, _p(step), rank, world,
                                                   timeout_ns, _p(status), _stream(stream), int(pdl)))


def linear_host(kind, w, scale, h_x, h_y, M, N, K, x_stage, y_stage, workspace=None, ws_size=0, stream=None):
    _check(lib().mc_sm100_linear_host(kind, _p(w), _p(scale), _p(h_x), _p(h_y), M, N, K, _p(x_stage),
                                      _p(y_stage), _p(workspace), ws_size, _stream(stream)))


def debug_set_math(bf16_math=-1, fp8_math=-1):
    lib().mc_sm100_debug_set_math(bf16_math, fp8_math)


def hint_next_weights(w, nbytes=None):
    """Names the weights the launch AFTER the next one streams (L2 prefetch); None clears the hint."""
    if w is None:
        lib().mc_sm100_hint_next_weights(None, 0)
    else:
        lib().mc_sm100_hint_next_weights(_p(w), int(nbytes if nbytes is not None else w.numel() * w.element_size()))


def debug_mma_rows_plan(n: int, sms: int = 148):
    """(block rows, blocks a CTA holds at a time, rows the fullest SM walks through) -- host logic only."""
    a, b, c = _u32(0), _u32(0), _u32(0)
    lib().mc_sm100_debug_mma_rows_plan(n, sms, C.byref(a), C.byref(b), C.byref(c))
    return a.value, b.value, c.value


def debug_chain_plan(fp8: bool, hidden: int, inter: int):
    """(slot bytes, rows per slot for K = hidden, for the gate_up pairs, for down) of the persistent M = 1 kernel -- host logic only."""
    v = [_u32(0) for _ in range(4)]
    lib().mc_sm100_debug_chain_plan(1 if fp8 else 0, hidden, inter, *[C.byref(x) for x in v])
    return tuple(x.value for x in v)


def debug_set_mma_rows(max_m: int) -> None:
    """bf16 batched linears up to max_m rows on the register-streaming mma.sync kernel (default 8; 0: tcgen05 only)."""
    lib().mc_sm100_debug_set_mma_rows(max_m)


def debug_set_chain(on: bool) -> None:
    """M = 1 steps of a one-GPU stack as one persistent kernel, or (default) one kernel per linear."""
    lib().mc_sm100_debug_set_chain(1 if on else 0)


def debug_set_prefetch(mode=-1, chunk_bytes=-1, evict_first=-1, cap_bytes=0):
    lib().mc_sm100_debug_set_prefetch(mode, chunk_bytes, evict_first, cap_bytes)


def debug_take_error() -> int:
    return lib().mc_sm100_debug_take_error()


# ---- decode stack ---------------------------------------------------------------------------
class StackDesc(C.Structure):
    _fields_ = [("struct_size", _u32), ("layers", _u32), ("hidden", _u32), ("qkv_rows", _u32), ("inter", _u32),
                ("vocab", _u32), ("precision", _u32), ("max_batch", _u32), ("eps", C.c_float),
                ("enable_cuda_graph", _u32), ("world", _u32), ("rank", _u32), ("reserved", _u32 * 2)]


SEC = {"qkv": 0, "o": 1, "gate_up": 2, "down": 3, "norm1": 4, "norm2": 5, "qkv_scale": 6, "o_scale": 7,
       "gate_up_scale": 8, "down_scale": 9, "lm_head": 10, "final_norm": 11, "lm_head_scale": 12}


def stack_desc(layers, hidden, qkv_rows, inter, vocab, fp8=False, max_batch=1, eps=1e-6, graph=True,
               world=1, rank=0) -> StackDesc:
    d = StackDesc()
    d.world, d.rank = (world if world > 1 else 0), rank
    d.struct_size = C.sizeof(StackDesc)
    d.layers, d.hidden, d.qkv_rows, d.inter, d.vocab = layers, hidden, qkv_rows, inter, vocab
    d.precision, d.max_batch, d.eps, d.enable_cuda_graph = (2 if fp8 else 0), max_batch, eps, int(graph)
    return d


def stack_sizes(desc):
    w, s = C.c_uint64(), C.c_uint64()
    _check(lib().mc_sm100_stack_sizes(C.byref(desc), C.byref(w), C.byref(s)))
    return w.value, s.value


def stack_section(desc, layer, which):
    off, n = C.c_uint64(), C.c_uint64()
    _check(lib().mc_sm100_stack_section(C.byref(desc), layer, SEC[which] if isinstance(which, str) else which,
                                        C.byref(off), C.byref(n)))
    return off.value, n.value


def stack_create(desc, weights, scratch):
    h = _vp()
    _check(lib().mc_sm100_stack_create(C.byref(desc), _p(weights), _p(scratch), C.byref(h)))
    return h


def stack_destroy(handle):
    lib().mc_sm100_stack_destroy(handle)


def stack_step(handle, x, M, tokens, stream=None):
    _check(lib().mc_sm100_stack_step(handle, _p(x), M, _p(tokens), _stream(stream)))


def stack_step_host(handle, h_x, M, h_tokens, stream=None):
    _check(lib().mc_sm100_stack_step_host(handle, _p(h_x), M, _p(h_tokens), _stream(stream)))


def stack_logits_ptr(handle) -> int:
    return lib().mc_sm100_stack_logits(handle)


def stack_exchange_bytes(desc) -> int:
    n = C.c_uint64()
    _check(lib().mc_sm100_stack_exchange_bytes(C.byref(desc), C.byref(n)))
    return n.value


def stack_bind_exchange(handle, peer_addrs, timeout_ns=0, stream=None):
    arr = (C.c_uint64 * len(peer_addrs))(*[int(a) for a in peer_addrs])
    _check(lib().mc_sm100_stack_bind_exchange(handle, C.cast(arr, _vp), timeout_ns, _stream(stream)))


def stack_exchange_status(handle, stream=None) -> int:
    v = _i32()
    _check(lib().mc_sm100_stack_exchange_status(handle, C.byref(v), _stream(stream)))
    return v.value


# ---- sharded linears (exchange inside the GEMV) -------------------------------------------------
class ShardIO(C.Structure):
    _fields_ = [("struct_size", _u32), ("world", _u32), ("rank", _u32), ("in_tagged", _u32), ("in_seq_mul", _u32),
                ("in_seq_add", _u32), ("out_slot", _u32), ("out_seq_mul", _u32), ("out_seq_add", _u32), ("reserved", _u32),
                ("d_step", _vp), ("d_status", _vp), ("timeout_ns", C.c_uint64), ("out_peer", C.c_uint64 * 8)]


def shard_io(world, rank, step, status, in_seq=None, out_slot=0, out_seq=None, out_peer=(), timeout_ns=0) -> ShardIO:
    """step/status: device tensors (or addresses); in_seq/out_seq: (mul, add) of the consumed / produced
    exchange, None = local input / local output; out_peer: address of every rank's gathered vector."""
    io = ShardIO()
    io.struct_size = C.sizeof(ShardIO)
    io.world, io.rank, io.out_slot = world, rank, out_slot
    if in_seq is not None:
        io.in_tagged, io.in_seq_mul, io.in_seq_add = 1, in_seq[0], in_seq[1]
    if out_seq is not None:
        io.out_seq_mul, io.out_seq_add = out_seq
    io.d_step, io.d_status, io.timeout_ns = _p(step), _p(status), timeout_ns
    for i, a in enumerate(out_peer):
        io.out_peer[i] = int(a)
    return io


def gemv_sharded(prologue, epilogue, w, scale, x, addend, norm_w, res_out, y, N, K, eps, io, stream=None, pdl=False):
    _check(lib().mc_sm100_gemv_sharded(prologue, epilogue, _p(w), _p(scale), _p(x), _p(addend), _p(norm_w), _p(res_out),
                                       _p(y), N, K, eps, C.cast(C.byref(io), _vp), _stream(stream), int(pdl)))


def lm_head_argmax_sharded(w, scale, res_in, addend, norm_w, res_out, logits, N, n, eps, index_base, stage, out_idx,
                           out_val, io, stream=None, pdl=False):
    _check(lib().mc_sm100_lm_head_argmax_sharded(_p(w), _p(scale), _p(res_in), _p(addend), _p(norm_w), _p(res_out),
                                                 _p(logits), N, n, eps, index_base, _p(stage), _p(out_idx), _p(out_val),
                                                 C.cast(C.byref(io), _vp), _stream(stream), int(pdl)))


def peer_argmax(val, idx, pair_peers, flag_peers, my_pairs, my_flags, step, rank, world, status, token, token_val=None,
                timeout_ns=0, stream=None, pdl=False, n_rows=1):
    _check(lib().mc_sm100_peer_argmax(_p(val), _p(idx), n_rows, _p(pair_peers), _p(flag_peers), _p(my_pairs), _p(my_flags),
                                      _p(step), rank, world, timeout_ns, _p(status), _p(token), _p(token_val),
                                      _stream(stream), int(pdl)))


# ---- packed weight file -----------------------------------------------------------------------
class WpkSection(C.Structure):
    _fields_ = [("name_hash", C.c_uint64), ("dtype", _u32), ("layout", _u32), ("rank", _u32), ("dims", _u32 * 8),
                ("data_offset", C.c_uint64), ("data_bytes", C.c_uint64), ("scale_offset", C.c_uint64),
                ("scale_bytes", C.c_uint64)]


def wpk_open(path: str):
    h = _vp()
    _check(lib().mc_sm100_wpk_open(path.encode(), C.byref(h)))
    return h


def wpk_close(h):
    lib().mc_sm100_wpk_close(h)


def wpk_find(h, name: str) -> WpkSection:
    sec = WpkSection()
    _check(lib().mc_sm100_wpk_find(h, name.encode(), C.byref(sec)))
    return sec


def wpk_write(path: str, sections, target_sm: int = 120) -> None:
    """sections: list of (name, bf16 uint16 array) or (name, e4m3 uint8 array, fp32 row scales); numpy arrays."""
    import numpy as np
    w = _vp()
    _check(lib().mc_sm100_wpk_writer_create(path.encode(), len(sections), target_sm, None, C.byref(w)))
    try:
        for sec in sections:
            name, arr = sec[0], np.ascontiguousarray(sec[1])
            dims = (C.c_uint32 * arr.ndim)(*arr.shape)
            sc = np.ascontiguousarray(sec[2], dtype=np.float32) if len(sec) == 3 else None
            _check(lib().mc_sm100_wpk_writer_add(w, name.encode(), 2 if sc is not None else 0, arr.ndim, C.cast(dims, _vp),
                                                 arr.ctypes.data, sc.ctypes.data if sc is not None else None))
    except Exception:
        lib().mc_sm100_wpk_writer_abort(w)
        raise
    _check(lib().mc_sm100_wpk_writer_finish(w))


def quantize_rows_host(w_u16):
    """bf16 weight [N, K] (numpy uint16) -> (e4m3 codes uint8 [N, K], fp32 row scales [N]) on the host."""
    import numpy as np
    w = np.ascontiguousarray(w_u16, dtype=np.uint16)
    q = np.empty(w.shape, dtype=np.uint8)
    sc = np.empty(w.shape[0], dtype=np.float32)
    _check(lib().mc_sm100_quantize_rows_host(w.ctypes.data, w.shape[0], w.shape[1], q.ctypes.data, sc.ctypes.data))
    return q, sc


def e4m3_from_f32_host(values):
    import numpy as np
    v = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty(v.shape, dtype=np.uint8)
    _check(lib().mc_sm100_e4m3_from_f32_host(v.ctypes.data, v.size, out.ctypes.data))
    return out


def wpk_upload(h, name, row_lo, row_hi, interleave, dst, scale_dst=None, stream=None):
    _check(lib().mc_sm100_wpk_upload(h, name.encode(), row_lo, row_hi, int(interleave), _p(dst),
                                     dst.numel() * dst.element_size(), _p(scale_dst), _stream(stream)))


def peer_allgather_rows(shard, rows, row_bytes, dst_pitch_bytes, slot_bytes, peer_bufs, peer_flags, my_flags, epoch, rank, world,
                        timeout_ns=0, status=None, stream=None, pdl=False):
    _check(lib().mc_sm100_peer_allgather_rows(_p(shard), rows, row_bytes, dst_pitch_bytes, slot_bytes, _p(peer_bufs), _p(peer_flags),
                                              _p(my_flags), _p(epoch), rank, world, timeout_ns, _p(status),
                                              _stream(stream), int(pdl)))


def peer_allgather(shard, shard_bytes, slot_bytes, peer_bufs, peer_flags, my_flags, epoch, rank, world,
                   timeout_ns=0, status=None, stream=None, pdl=False):
    _check(lib().mc_sm100_peer_allgather(_p(shard), shard_bytes, slot_bytes, _p(peer_bufs), _p(peer_flags),
                                         _p(my_flags), _p(epoch), rank, world, timeout_ns, _p(status),
                                         _stream(stream), int(pdl)))


# ---- model / session / batch group (include/mc_sm100a_runtime.h) --------------------------------
ABI_VERSION = 0x00020000


class ModelOptions(C.Structure):
    _fields_ = [("struct_size", _u32), ("abi_version", _u32), ("device_id", _i32), ("max_sessions", _u32), ("precision", _u32),
                ("enable_cuda_graph", _u32), ("synth_layers", _u32), ("synth_hidden", _u32), ("synth_qkv_rows", _u32),
                ("synth_inter", _u32), ("synth_vocab", _u32), ("reserved0", _u32), ("synth_seed", C.c_uint64), ("reserved", _u32 * 4)]


class GenerationConfig(C.Structure):
    _fields_ = [("struct_size", _u32), ("max_new_tokens", _u32), ("temperature", C.c_float), ("top_p", C.c_float), ("top_k", _u32),
                ("repetition_penalty", C.c_float), ("seed", C.c_uint64)]


class RuntimeStats(C.Structure):
    _fields_ = [("prompt_tokens", C.c_uint64), ("generated_tokens", C.c_uint64), ("prefill_us", C.c_uint64), ("decode_us", C.c_uint64),
                ("peak_vram_bytes", C.c_uint64), ("cuda_graph_launches", C.c_uint64)]


class BatchOptions(C.Structure):
    _fields_ = [("struct_size", _u32), ("abi_version", _u32), ("max_slots", _u32), ("max_context_tokens", _u32), ("reserved", _u32 * 4)]


def model_options(fp8=False, max_sessions=8, graph=True, device=0, synth=None, seed=1) -> ModelOptions:
    o = ModelOptions()
    o.struct_size, o.abi_version, o.device_id, o.max_sessions = C.sizeof(ModelOptions), ABI_VERSION, device, max_sessions
    o.precision, o.enable_cuda_graph, o.synth_seed = (2 if fp8 else 0), int(graph), seed
    if synth is not None:
        o.synth_layers, o.synth_hidden, o.synth_qkv_rows, o.synth_inter, o.synth_vocab = synth
    return o


def greedy_config(max_new_tokens=16) -> GenerationConfig:
    g = GenerationConfig()
    g.struct_size, g.max_new_tokens, g.top_k, g.repetition_penalty = C.sizeof(GenerationConfig), max_new_tokens, 1, 1.0
    return g


def model_load(model_dir: str, options: ModelOptions):
    h = _vp()
    _check(lib().mc_sm100_model_load(model_dir.encode(), C.cast(C.byref(options), _vp), C.byref(h)))
    return h


def model_destroy(model):
    lib().mc_sm100_model_destroy(model)


def model_dims(model):
    v = [_u32() for _ in range(5)]
    _check(lib().mc_sm100_debug_model_dims(model, *[C.byref(x) for x in v]))
    return tuple(x.value for x in v)


def session_create(model):
    h = _vp()
    _check(lib().mc_sm100_session_create(model, C.byref(h)))
    return h


def session_reset(session):
    _check(lib().mc_sm100_session_reset(session))


def session_destroy(session):
    lib().mc_sm100_session_destroy(session)


def prefill(session, token_ids):
    arr = (_i32 * len(token_ids))(*token_ids)
    _check(lib().mc_sm100_prefill(session, C.cast(arr, _vp), len(token_ids)))


def decode_one(session, config: GenerationConfig) -> int:
    tok = _i32(-1)
    _check(lib().mc_sm100_decode_one(session, C.cast(C.byref(config), _vp), C.byref(tok)))
    return tok.value


def get_stats(session) -> RuntimeStats:
    st = RuntimeStats()
    _check(lib().mc_sm100_get_stats(session, C.cast(C.byref(st), _vp)))
    return st


def session_logits(session, count):
    import numpy as np
    out = np.empty(count, dtype=np.uint16)
    _check(lib().mc_sm100_debug_session_logits(session, out.ctypes.data, count))
    return out


def batch_group_create(model, max_slots, max_context_tokens=0):
    o = BatchOptions()
    o.struct_size, o.abi_version, o.max_slots, o.max_context_tokens = C.sizeof(BatchOptions), ABI_VERSION, max_slots, max_context_tokens
    h = _vp()
    _check(lib().mc_sm100_batch_group_create(model, C.cast(C.byref(o), _vp), C.byref(h)))
    return h


def batch_group_add(group, session) -> int:
    slot = _u32(0xFFFFFFFF)
    _check(lib().mc_sm100_batch_group_add(group, session, C.byref(slot)))
    return slot.value


def batch_group_remove(group, slot):
    _check(lib().mc_sm100_batch_group_remove(group, slot))


def batch_step(group, slot_ids, configs):
    n = len(slot_ids)
    ids = (_u32 * n)(*slot_ids)
    cfgs = (GenerationConfig * n)(*configs)
    out = (_i32 * n)()
    _check(lib().mc_sm100_batch_step(group, C.cast(ids, _vp), n, C.cast(cfgs, _vp), C.cast(out, _vp)))
    return list(out)


def batch_group_destroy(group):
    lib().mc_sm100_batch_group_destroy(group)


def batch_group_stats(group):
    steps, us, members, graphs = C.c_uint64(), C.c_uint64(), _u32(), _u32()
    _check(lib().mc_sm100_debug_batch_group_stats(group, C.byref(steps), C.byref(us), C.byref(members), C.byref(graphs)))
    return {"steps": steps.value, "decode_us": us.value, "members": members.value, "graphs": graphs.value}
