"""ctypes binding of the kernel library.

Every launcher is a plain C function over raw device pointers and a stream
(see csrc/common.cuh).  This module loads the library, declares the argument
types once and turns a non-zero return into an exception.  There is no CPU
fallback: if the library cannot be built or loaded, using an op raises.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Dict, Optional

from . import build as _build

c_int, c_float, c_ll, c_vp = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p

# name -> argument types (all return int)
_SIGNATURES: Dict[str, list] = {
    "qnn_embed": [c_vp, c_vp, c_int, c_float, c_vp, c_int, c_int, c_int, c_vp],
    "qnn_embed_rmsnorm": [c_vp, c_vp, c_int, c_float, c_vp, c_vp, c_int, c_float, c_int, c_vp, c_int, c_int, c_int, c_int,
                          c_vp],
    "qnn_rmsnorm": [c_vp, c_int, c_vp, c_int, c_float, c_int, c_vp, c_int, c_int, c_int, c_vp],
    "qnn_add_rmsnorm": [c_vp, c_vp, c_int, c_vp, c_int, c_float, c_int, c_vp, c_int, c_float, c_int,
                        c_vp, c_int, c_int, c_int, c_vp],
    "qnn_add": [c_vp, c_vp, c_int, c_ll, c_vp],
    "qnn_gated_act": [c_vp, c_vp, c_int, c_int, c_int, c_int, c_vp],
    "qnn_softcap": [c_vp, c_int, c_vp, c_float, c_ll, c_vp],
    "qnn_gather_rows": [c_vp, c_int, c_vp, c_vp, c_int, c_int, c_int, c_vp],
    "qnn_cast": [c_vp, c_int, c_vp, c_int, c_ll, c_vp],
    "qnn_check_finite": [c_vp, c_ll, c_vp, c_vp],
    "qnn_rope_cache_write": [c_vp, c_int, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp,
                             c_vp, c_int, c_int, c_int, c_vp, c_int, c_vp],
    "qnn_skinny_bf16": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_vp],
    "qnn_skinny_argmax": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_float, c_vp, c_vp],
    "qnn_skinny_qkv_rope": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                            c_int, c_int, c_int, c_vp, c_int, c_vp],
    "qnn_linear_bf16_any": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_vp],
    "qnn_gemv_f32": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_float, c_int, c_vp],
    "qnn_sgemm_f32": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_float, c_vp],
    "qnn_gemm_tcgen05": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp],
    "qnn_gemm_tcgen05_2cta": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp],
    "qnn_gemm_skinny_tcgen05": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_float, c_int, c_vp, c_vp],
    "qnn_gemm_skinny_tcgen05_argmax": [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_float, c_vp, c_vp, c_vp],
    "qnn_attn_decode": [c_vp, c_ll, c_int, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_vp, c_int, c_int,
                        c_int, c_int, c_float, c_float, c_int, c_vp, c_vp, c_int, c_vp, c_ll, c_vp],
    "qnn_attn_extend": [c_vp, c_vp, c_vp, c_ll, c_int, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_ll, c_vp, c_vp,
                        c_vp, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_vp],
    "qnn_attn_supports": [c_int, c_int, c_int, c_int],
    "qnn_attn_prefill_generic": [c_vp, c_vp, c_vp, c_ll, c_int, c_vp, c_ll, c_vp, c_vp, c_int, c_int, c_int,
                                 c_int, c_float, c_float, c_int, c_vp],
    "qnn_attn_prefill_mma": [c_vp, c_vp, c_vp, c_ll, c_vp, c_ll, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int,
                             c_float, c_float, c_int, c_vp],
    "qnn_attn_prefill_tcgen05": [c_vp, c_ll, c_vp, c_ll, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_float,
                                 c_float, c_int, c_vp, c_vp],
    "qnn_attn_extend_gather": [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int,
                               c_int, c_int, c_int, c_int, c_vp],
    "qnn_attn_prefill_paged": [c_vp, c_ll, c_int, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_ll, c_vp, c_vp,
                               c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_vp],
    "qnn_sample": [c_vp, c_int, c_int, c_int, c_float, c_float, c_float, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                   c_vp, c_vp],
    "qnn_sample_candidates": [c_vp, c_int, c_int, c_int, c_int, c_float, c_float, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                              c_vp],
    "qnn_sample_scratch_bytes": [c_int, c_int, c_int],
    "qnn_mark_seen": [c_vp, c_vp, c_vp, c_int, c_int, c_vp],
}

ERR_UNSUPPORTED, ERR_ARGUMENT = 10001, 10002


class KernelError(RuntimeError):
    pass


class NonFiniteLogits(RuntimeError):
    """NaN or Inf in the logits of a forward pass (the reference flags them after every forward,
    src/models/QuickNN.Models.Gemma2.pas:196, and raises "non-finite values" at the next readback,
    QuickNN.Vulkan.Context.Implementation.inc:732-756)."""


_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_path: Optional[str] = None


def load() -> ctypes.CDLL:
    """Build if needed, then load.  Raises if that is impossible."""
    global _lib, _path
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.build()
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"the kernel library {path} could not be loaded: {e}") from None
        for name, args in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                raise KernelError(f"the kernel library {path} lacks the entry point {name}") from None
            fn.argtypes = args
            fn.restype = c_int
        lib.cudaGetErrorString_qnn = None
        _lib, _path = lib, path
    return _lib


def library_file() -> Optional[str]:
    return _path


launches = 0          # kernels launched through this module since import (a graph replay is not seen here)


def check(code: int, what: str, kernels: int = 1) -> None:
    global launches
    if code == 0:
        launches += kernels
        return
    if code == ERR_UNSUPPORTED:
        raise KernelError(f"{what}: the kernel does not take these sizes")
    if code == ERR_ARGUMENT:
        raise KernelError(f"{what}: invalid argument (alignment, divisibility or range)")
    raise KernelError(f"{what}: CUDA error {code} at launch")
