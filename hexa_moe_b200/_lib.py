"""ctypes binding of libhexa_moe_b200.so (the C ABI declared in include/hexa_moe_b200.h).

The library is the only execution path: there is no CPU or PyTorch fallback.  `lib()` raises
if the shared object is missing; every wrapper raises `HexaError` on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhexa_moe_b200.so")

F32, F16, BF16 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3, 4
B_NK, B_KN = 0, 1
EPI_LINEAR, EPI_ACT, EPI_DACT = 0, 1, 2
ENGINE_AUTO, ENGINE_TCGEN05, ENGINE_SIMT = 0, 1, 2
ROW_TILE = 128

_DT = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

i32p, vp, i64, ci, sz = C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_size_t

# name -> (restype, argtypes); mirrors include/hexa_moe_b200.h one to one
SIGNATURES = {
    "hexa_version": (ci, []),
    "hexa_last_error_string": (C.c_char_p, []),
    "hexa_set_status_word": (ci, [vp]),
    "hexa_pending_device_status": (ci, []),
    "hexa_set_wait_limit_ns": (ci, [C.c_uint64]),
    "hexa_set_tc_debug": (ci, [ci]),
    "hexa_set_sm_limit": (ci, [ci]),
    "hexa_route_row_capacity": (i64, [i64, ci, ci, ci]),
    "hexa_route_workspace_bytes": (sz, [i64, ci, ci]),
    "hexa_route_pair_capacity": (i64, [i64, ci, ci]),
    "hexa_route": (ci, [vp, i64, ci, i64, i64, ci, ci, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "hexa_gather_rows": (ci, [vp, i64, vp, vp, ci, i64, i64, vp, i64, ci, vp]),
    "hexa_combine_rows": (ci, [vp, i64, vp, i64, ci, i64, vp, i64, ci, vp]),
    "hexa_esmm": (ci, [vp, i64, vp, ci, i64, i64, vp, i64, vp, i64, vp, i64, vp, vp, vp, vp, ci, i64, i64, i64, ci, ci, ci, ci, vp]),
    "hexa_esmm_experts": (ci, [vp, i64, vp, ci, i64, i64, vp, i64, vp, i64, vp, i64, vp, vp, vp, vp, ci, i64, i64, i64, ci, ci, ci, ci,
                               ci, ci, vp]),
    "hexa_esmm_ess": (ci, [vp, i64, vp, ci, i64, i64, vp, i64, vp, i64, vp, i64, vp, vp, vp, vp, ci, i64, i64, i64, ci, ci, ci, ci,
                           vp, i64, vp, sz, vp]),
    "hexa_estmm_workspace_bytes": (sz, [ci, i64, i64, i64, ci]),
    "hexa_estmm": (ci, [vp, i64, vp, i64, vp, ci, i64, i64, i64, vp, i64, i64, i64, i64, ci, ci, ci, ci, vp, sz, vp]),
    "hexa_estmm_scatter": (ci, [vp, i64, vp, i64, vp, ci, i64, i64, i64, vp, ci, i64, i64, i64, ci, ci, vp]),
    "hexa_copy_2d": (ci, [vp, i64, vp, i64, i64, i64, vp]),
    "hexa_stream_wait_value": (ci, [vp, C.c_int32, vp]),
    "hexa_mean_slices": (ci, [vp, vp, ci, i64, ci, vp, ci, vp]),
    "hexa_ess_workspace_bytes": (sz, [i64, i64]),
    "hexa_ess": (ci, [vp, i64, vp, ci, i64, i64, vp, i64, ci, vp, sz, vp]),
    "hexa_mask_pad_rows": (ci, [vp, i64, vp, vp, ci, i64, i64, ci, vp]),
    "hexa_gate_max_experts": (ci, []),
    "hexa_gate_workspace_bytes": (sz, []),
    "hexa_gate_topk": (ci, [vp, i64, i64, ci, ci, vp, vp, vp, vp, vp, sz, vp]),
    "hexa_gate_loss_grad": (ci, [vp, i64, i64, ci, vp, vp, vp, i64, vp]),
    "hexa_gate_topk_load_importance": (ci, [vp, vp, i64, i64, ci, ci, C.c_float, vp, vp, vp, vp, vp, sz, vp]),
    "hexa_gate_load_importance_grad": (ci, [vp, vp, i64, i64, ci, ci, C.c_float, vp, vp, vp, vp, i64, vp]),
    "hexa_ess_static_capacity_bytes": (sz, []),
    "hexa_ess_static": (ci, [vp, i64, vp, ci, i64, i64, vp, i64, ci, vp]),
}

_lock = threading.Lock()
_lib = None


class HexaError(RuntimeError):
    pass


def lib():
    """Load the shared library once.  Fails loudly if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise HexaError(
                        f"{LIB_PATH} is missing: build it with `python -m hexa_moe_b200.build` "
                        "(there is no fallback path)")
                handle = C.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)      # AttributeError if the symbol is not exported
                    fn.restype, fn.argtypes = res, args
                _lib = handle
    return _lib


ERR_DEVICE = -5
_STATUS_CODES = {1: "the TMA producer waited for a free ring slot", 2: "the MMA issuer waited for a drained accumulator",
                 3: "the MMA issuer waited for operands", 4: "an epilogue warp waited for an accumulator"}


def check(status: int, what: str):
    """Raise on a non-zero return code, and on a code that a kernel launched earlier left in the device's status
    word (a bounded wait that ran out): the host sees it at its next call into the library, without synchronising."""
    if status != 0:
        raise HexaError(f"{what} failed ({status}): {lib().hexa_last_error_string().decode()}")
    if _status_words:
        code = lib().hexa_pending_device_status()
        if code:
            raise HexaError(f"{what}: a kernel on this device gave up a bounded wait (status code {code}: "
                            f"{_STATUS_CODES.get(code, 'unknown')}); results since then are incomplete ({ERR_DEVICE})")


# One status word per device in pinned host memory: kernels store a code there when a wait inside them runs out,
# the host reads it without a copy.  Installed the first time an operator runs on a device.
_status_words = {}


def ensure_status_word(device_index: int):
    w = _status_words.get(device_index)
    if w is None:
        lib()                      # loaded before the lock is taken: lib() takes the same (non-reentrant) lock
        with _lock:
            w = _status_words.get(device_index)
            if w is None:
                w = torch.zeros(1, dtype=torch.int32).pin_memory()
                with torch.cuda.device(device_index):
                    rc = lib().hexa_set_status_word(w.data_ptr())
                if rc != 0:
                    raise HexaError(f"hexa_set_status_word failed ({rc}): {lib().hexa_last_error_string().decode()}")
                _status_words[device_index] = w
    return w


def device_status(device_index: int = None) -> int:
    """Code in the status word of a device (0: no kernel has reported a failure)."""
    idx = torch.cuda.current_device() if device_index is None else device_index
    w = _status_words.get(idx)
    return 0 if w is None else int(w[0])


def clear_device_status(device_index: int = None):
    idx = torch.cuda.current_device() if device_index is None else device_index
    w = _status_words.get(idx)
    if w is not None:
        w.zero_()


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise HexaError(f"unsupported dtype {t.dtype}")


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise HexaError("hexa_moe_b200 operators run on CUDA tensors only (no CPU path)")
    idx = t.device.index
    if idx not in _status_words:
        ensure_status_word(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(t.device).cuda_stream
