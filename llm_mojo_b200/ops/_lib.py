"""ctypes binding of ``csrc/libllmb200.so``.

The library exports plain C functions that take raw device pointers and a stream and return
a CUDA error code.  ``lib()`` raises if the shared object is missing: on a GPU box a silent
fallback to PyTorch ops would hide a broken build.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
# LLMB_BOUNDS_CHECK=1 loads the checked build (data-dependent indices tested before use; see csrc/common.cuh)
BOUNDS_CHECK = os.environ.get("LLMB_BOUNDS_CHECK", "") not in ("", "0")
_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc",
                         "libllmb200_check.so" if BOUNDS_CHECK else "libllmb200.so")

c_int, c_ll, c_f, c_p, c_ull = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p, ctypes.c_ulonglong

_SIGS = {
    "llmb_encoder_fwd": [c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_int, c_p],
    "llmb_encoder_bwd_scratch_bytes": [c_int, c_int],
    "llmb_encoder_bwd": [c_p, c_p, c_p, c_p, c_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_p],
    "llmb_bounds_report_elementwise": [c_p, c_int],
    "llmb_bounds_report_classifier": [c_p, c_int],
    "llmb_gelu_fwd": [c_p, c_p, c_ll, c_int, c_p],
    "llmb_gelu_bwd": [c_p, c_p, c_p, c_ll, c_int, c_p],
    "llmb_dbias_scratch_bytes": [c_int, c_int],
    "llmb_dbias": [c_p, c_p, c_p, c_ll, c_int, c_int, c_int, c_p],
    "llmb_cast_f32_to_bf16": [c_p, c_p, c_ll, c_p],
    "llmb_nan_census": [c_p, c_p, c_ll, c_int, c_p],
    "llmb_layernorm_fwd": [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_p],
    "llmb_layernorm_bwd_scratch_bytes": [c_int, c_int],
    "llmb_layernorm_bwd": [c_p, c_p, c_p, c_p, c_ll, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_p],
    "llmb_layernorm_bwd_colsum": [c_p, c_p, c_p, c_p, c_p, c_ll, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_p],
    "llmb_fused_classifier": [c_p, c_p, c_p, c_f, c_int, c_int, c_int, c_int, c_int, c_p, c_p],
    "llmb_ce_pass1": [c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_p],
    "llmb_ce_loss": [c_p, c_p, c_int, c_p],
    "llmb_ce_pass2": [c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_int, c_f, c_int, c_p],
    "llmb_softmax_rows": [c_p, c_p, c_int, c_int, c_int, c_f, c_int, c_p],
    "llmb_softmax_bwd": [c_p, c_p, c_p, c_int, c_int, c_int, c_p],
    "llmb_crossentropy_fwd": [c_p, c_p, c_p, c_int, c_int, c_p],
    "llmb_crossentropy_bwd": [c_p, c_p, c_p, c_p, c_int, c_int, c_p],
    "llmb_adamw": [c_p, c_p, c_p, c_p, c_p, c_ll, c_f, c_f, c_f, c_f, c_f, c_f, c_p, c_int, c_ull, c_int, c_int, c_p],
    "llmb_norm_sq_blocks": [],
    "llmb_global_norm_sq": [c_p, c_p, c_ll, c_p, c_int, c_p],
    "llmb_sr_cast_bf16": [c_p, c_p, c_ll, c_ull, c_p],
    "llmb_gemm": [c_p, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_int, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_p, c_p],
    "llmb_gemm_nvfp4": [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_ll, c_ll, c_int, c_int, c_p, c_p],
    "llmb_gemm_mxfp8": [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_int, c_int, c_p, c_p],
    "llmb_fp8_block_quant": [c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_int, c_p],
    "llmb_gemm_set_colsum": [c_p],
    "llmb_gemm_debug_mn_strides": [c_int, c_int],
    "llmb_gemm_set_pair_mode": [c_int],
    "llmb_amax": [c_p, c_p, c_ll, c_int, c_p],
    "llmb_amax_rht": [c_p, c_p, c_int, c_int, c_int, c_int, c_p],
    "llmb_fp8_block_fake_quant": [c_p, c_p, c_int, c_int, c_int, c_int, c_p],
    "llmb_amax_state_floats": [],
    "llmb_amax_update": [c_p, c_p, c_f, c_f, c_p],
    "llmb_quantize_fp8": [c_p, c_p, c_p, c_ll, c_int, c_int, c_p],
    "llmb_quantize_fp8_delayed": [c_p, c_p, c_p, c_p, c_ll, c_int, c_f, c_f, c_int, c_p],
    "llmb_fp8_block_quant_dual": [c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_p],
    "llmb_fp8_prepare": [c_p, c_p, c_f, c_f, c_p, c_p, c_f, c_f, c_p, c_p, c_p, c_p, c_p, c_p, c_p],
    "llmb_fp8_push": [c_p, c_p, c_p, c_p, c_p],
    "llmb_quantize_fp8_amax": [c_p, c_p, c_p, c_p, c_ll, c_int, c_int, c_p],
    "llmb_dequantize_fp8": [c_p, c_p, c_p, c_ll, c_int, c_p],
    "llmb_nvfp4_tensor_scale": [c_p, c_p, c_p],
    "llmb_nvfp4_scale_bytes": [c_ll, c_ll, c_int],
    "llmb_nvfp4_quantize": [c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_int, c_int, c_ull, c_ull, c_ll, c_int,
                            c_int, c_p],
    "llmb_nvfp4_dequantize": [c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_p],
    "llmb_hadamard16": [c_p, c_p, c_ll, c_int, c_int, c_p],
    "llmb_rng_uniform": [c_p, c_ll, c_ull, c_ull, c_ull, c_p],
    "llmb_attention_fwd": [c_p, c_p, c_p, c_int, c_int, c_int, c_p, c_p],
    "llmb_attention_bwd": [c_p, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_p, c_p],
    "llmb_attention_bwd_dbias": [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_p, c_p],
    "llmb_attention_bwd_fused": [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_p, c_p],
    "llmb_attention_bwd_fused_stats_floats": [c_int, c_int, c_int],
    "llmb_attention_bwd_fused_acc_floats": [c_int, c_int, c_int],
}
_RET_LL = {"llmb_encoder_bwd_scratch_bytes", "llmb_dbias_scratch_bytes", "llmb_layernorm_bwd_scratch_bytes",
           "llmb_nvfp4_scale_bytes", "llmb_attention_bwd_fused_stats_floats", "llmb_attention_bwd_fused_acc_floats"}


def lib_path() -> str:
    return _LIB_PATH


def available() -> bool:
    return os.path.exists(_LIB_PATH)


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m llm_mojo_b200.build` "
                "(CUDA tensors never fall back to PyTorch ops)")
        L = ctypes.CDLL(_LIB_PATH)
        for name, sig in _SIGS.items():
            if not hasattr(L, name):
                continue
            fn = getattr(L, name)
            fn.argtypes = sig
            fn.restype = c_ll if name in _RET_LL else c_int
        _LIB = L
    return _LIB


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"unsupported dtype {t.dtype}")


class KernelError(RuntimeError):
    pass


def check(rc: int, name: str) -> None:
    if rc != 0:
        raise KernelError(f"{name} failed with code {rc}")


# A device-resident status word that kernels with bounded waits set on expiry.
_STATUS = {}


def status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[key] = t
    return t


SITES = {1: "encoder_fwd token id", 2: "encoder_bwd token id", 3: "fused_classifier target id", 4: "chunked CE target id"}


def bounds_report(reset: bool = True):
    """Checked build: the first out-of-range data-dependent index each kernel file saw since the last reset, as
    (site name, value, limit) tuples; empty when everything was in range (always empty in the normal build)."""
    out = []
    for name in ("llmb_bounds_report_elementwise", "llmb_bounds_report_classifier"):
        rec = (c_int * 4)()
        check(getattr(lib(), name)(rec, int(reset)), name)
        if rec[0]:
            out.append((SITES.get(rec[1], f"site {rec[1]}"), rec[2], rec[3]))
    return out


def read_status(device: Optional[torch.device] = None) -> int:
    """Synchronising read of the status word (0 = ok, 1 = a bounded wait expired)."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    return int(status_word(device).item())
