"""ctypes binding of ``lib/libfbam_kernels.so`` and ``lib/libfbam_kernels_fp16.so`` (hand-written sm_100a kernels).

The kernel sources are compiled twice, once per 16-bit element type (bf16, IEEE half; fp32 accumulation in both);
the two libraries export the same plain C entry points that take device pointers, sizes and a CUDA stream.
``lib(like)`` returns the library for the dtype of ``like``.  This module loads them, mirrors their parameter
structs, and converts non-zero return codes and device-side status words into Python exceptions.  If a library is
absent on a machine that has a GPU, loading raises — CUDA tensors never fall back to a PyTorch implementation
silently.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from ..utils import debug as _debug
from ..utils import plan as _plan

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libfbam_kernels.so")
LIB_PATH_FP16 = os.path.join(os.path.dirname(_HERE), "lib", "libfbam_kernels_fp16.so")
_lib: Optional[C.CDLL] = None
_lib_fp16: Optional[C.CDLL] = None
ELEM_DTYPES = (torch.bfloat16, torch.float16)

GEMM_ACT = {"none": 0, "gelu": 1, "relu": 2}
GEMM_ACC_NONE, GEMM_ACC_RMW, GEMM_ACC_ATOMIC = 0, 1, 2
_ERRORS = {1: "unsupported shape", 2: "operand not 16-byte aligned", 3: "tensor-map encode failed",
           4: "driver entry point unavailable", 5: "kernel launch failed",
           101: "TMA producer wait timed out", 102: "MMA wait timed out", 103: "epilogue wait timed out",
           201: "LSTM grid barrier timed out"}


class ConvGeom(C.Structure):
    _fields_ = [("batch", C.c_int), ("grid_h", C.c_int), ("grid_w", C.c_int),
                ("tn", C.c_int), ("th", C.c_int), ("tw", C.c_int),
                ("in_mul", C.c_int),
                ("out_mul", C.c_int), ("out_off_h", C.c_int), ("out_off_w", C.c_int), ("out_h", C.c_int), ("out_w", C.c_int),
                ("num_taps", C.c_int),
                ("tap_dh", C.c_int * 9), ("tap_dw", C.c_int * 9),
                ("c_blocks", C.c_int), ("tiles_w", C.c_int), ("tiles_h", C.c_int)]


class ConvClass(C.Structure):
    _fields_ = [("num_taps", C.c_int), ("tap_dh", C.c_int * 4), ("tap_dw", C.c_int * 4),
                ("out_off_h", C.c_int), ("out_off_w", C.c_int), ("k_block_base", C.c_int)]


class GemmParams(C.Structure):
    _fields_ = [("D", C.c_void_p), ("ldd", C.c_longlong),
                ("bias", C.c_void_p),
                ("residual", C.c_void_p), ("ldr", C.c_longlong),
                ("preact_out", C.c_void_p),
                ("gelu_grad_in", C.c_void_p),
                ("status", C.c_void_p),
                ("alpha", C.c_float),
                ("out_fp32", C.c_int), ("bias_fp32", C.c_int), ("act", C.c_int), ("accumulate", C.c_int),
                ("bn", C.c_int), ("bm", C.c_int), ("max_ctas", C.c_int), ("splits", C.c_int),
                ("split_workspace", C.c_void_p), ("split_stride", C.c_longlong),
                ("ready_flags", C.c_void_p), ("tile_m_rotate", C.c_int), ("flag_rows", C.c_int), ("flag_on_b", C.c_int),
                ("flag_epoch", C.c_uint), ("flag_spin_limit", C.c_uint),
                ("rs_out", C.c_void_p * 8), ("rs_rows_per_rank", C.c_int), ("rs_slot_plus1", C.c_int),
                ("rs_row_stores", C.c_int),
                ("ce_mode", C.c_int), ("ce_vocab", C.c_int), ("ce_slots", C.c_int), ("ce_scale", C.c_float),
                ("ce_partial", C.c_void_p), ("ce_tgt_logit", C.c_void_p), ("ce_lse", C.c_void_p),
                ("ce_targets", C.c_void_p),
                ("mode", C.c_int), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("tiles_m", C.c_int),
                ("k_blocks", C.c_int), ("a_mn_major", C.c_int), ("b_mn_major", C.c_int), ("vec_ok", C.c_int),
                ("conv", ConvGeom),
                ("num_classes", C.c_int), ("cls", ConvClass * 4),
                ("tma_store", C.c_int), ("st_bw", C.c_int), ("st_bh", C.c_int), ("st_bn", C.c_int)]


def available(dtype: torch.dtype = torch.bfloat16) -> bool:
    return os.path.exists(LIB_PATH_FP16 if dtype == torch.float16 else LIB_PATH)


def _check_struct_layout(library: C.CDLL, path: str) -> None:
    """The parameter struct is mirrored by hand above: refuse a library whose layout differs (a stale build)."""
    got = (C.c_longlong * 8)()
    library.fbam_gemm_params_layout.restype = None
    library.fbam_gemm_params_layout(got)
    mine = [C.sizeof(GemmParams), GemmParams.status.offset, GemmParams.split_workspace.offset,
            GemmParams.rs_out.offset, GemmParams.rs_row_stores.offset, GemmParams.mode.offset,
            GemmParams.conv.offset, C.sizeof(ConvGeom)]
    if list(got) != mine:
        raise RuntimeError(f"{path} was built from different sources than this binding (GemmParams layout "
                           f"{list(got)} vs {mine}); run `python -m fbamtrain_b200.build`")


def _load(path: str) -> C.CDLL:
    if not os.path.exists(path):
        raise RuntimeError(f"native kernel library missing: {path} (run `python -m fbamtrain_b200.build`)")
    library = C.CDLL(path)
    _check_struct_layout(library, path)
    for name in ("fbam_gemm", "fbam_conv", "fbam_conv_wgrad", "fbam_gemm2", "fbam_conv2",
                 "fbam_lstm_persistent_max_hidden", "fbam_lstm_fwd_ex", "fbam_lstm_bwd_ex", "fbam_elem_is_fp16"):
        getattr(library, name).restype = C.c_int
    return library


def lib(like=None) -> C.CDLL:
    """The kernel library for the 16-bit element type of ``like`` (a tensor or a dtype): the half-precision build
    for ``torch.float16``, the bf16 build for everything else (bf16, and calls whose operands are all fp32 or
    integer, which are the same code in both)."""
    global _lib, _lib_fp16
    dtype = like.dtype if isinstance(like, torch.Tensor) else like
    if dtype == torch.float16:
        if _lib_fp16 is None:
            _lib_fp16 = _load(LIB_PATH_FP16)
            if _lib_fp16.fbam_elem_is_fp16() != 1:
                raise RuntimeError(f"{LIB_PATH_FP16} was not built with half-precision elements")
        return _lib_fp16
    if _lib is None:
        _lib = _load(LIB_PATH)
        if _lib.fbam_elem_is_fp16() != 0:
            raise RuntimeError(f"{LIB_PATH} was not built with bf16 elements")
    return _lib


_launches = 0


def launches() -> int:
    """Number of native entry-point calls that launched kernels since import."""
    return _launches


def check(code: int, what: str) -> None:
    global _launches
    if code != 0:
        detail = ""
        if code in (3, 5):
            for loaded in (_lib, _lib_fp16):
                if loaded is not None and hasattr(loaded, "fbam_last_driver_error") and loaded.fbam_last_driver_error():
                    detail = (f"; driver result {loaded.fbam_last_driver_error()}, pending runtime error "
                              f"{loaded.fbam_pending_runtime_error()}")
        raise RuntimeError(f"{what}: {_ERRORS.get(code, 'error')} (code {code}){detail}")
    _launches += 1
    if _debug.BREAK_ON_LAUNCH and _debug.break_requested(_launches, what):
        breakpoint()      # FBAMTRAIN_BREAK_ON_LAUNCH: inspect the caller's frames ("up"), "c" continues
    recording = _plan.active()
    if recording is not None:
        recording.on_launch(what)


def stream_ptr() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


_status = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait expires."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


_status_probe = {}


def check_status_late(device: torch.device) -> None:
    """Raises if a kernel reported a timed-out wait, without draining the device: every call queues an asynchronous
    copy of the status word into pinned host memory and examines the copy queued by the PREVIOUS call (whose event has
    long completed by then).  A training loop calls this once per step; an expired wait therefore stops the run one
    step later instead of letting it train on through broken collectives."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    probe = _status_probe.get(key)
    if probe is None:
        probe = {"host": torch.zeros(1, dtype=torch.int32).pin_memory(), "event": None}
        _status_probe[key] = probe
    if probe["event"] is not None:
        probe["event"].synchronize()
        code = int(probe["host"][0])
        if code != 0:
            status_word(device).zero_()
            probe["event"] = None
            raise RuntimeError(f"device-side wait expired: {_ERRORS.get(code, 'error')} (code {code})")
    probe["host"].copy_(status_word(device), non_blocking=True)
    ev = torch.cuda.Event()
    ev.record()
    probe["event"] = ev


def check_status(device: torch.device) -> None:
    """Synchronises and raises if any kernel reported a timed-out wait since the last check."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise RuntimeError(f"device-side wait expired: {_ERRORS.get(code, 'error')} (code {code})")
