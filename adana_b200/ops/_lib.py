"""ctypes binding of the in-tree sm_100a kernel library (`adana_b200/lib/libadana_b200.so`).

The library exposes a plain C ABI (see `csrc/api.h`): raw device pointers plus the CUDA
stream.  Keeping torch headers out of the kernels makes a full rebuild take seconds.

On a machine with a GPU the library is required: `lib()` raises if it cannot be loaded,
so that no op silently falls back to a PyTorch implementation.  On a CPU-only machine
`available()` is False and the ops use their PyTorch reference paths.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

# ADANA_DEBUG=1 selects the checked build (`python -m adana_b200.build --debug`): kernels compare the indices they
# compute with their extents and report through the status word (csrc/common.cuh)
DEBUG_BUILD = os.environ.get("ADANA_DEBUG", "0") not in ("", "0")
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / ("libadana_b200_debug.so" if DEBUG_BUILD else "libadana_b200.so")
_DEBUG_UNITS = ("misc", "rope", "attention", "norm", "optim", "comm", "gemm", "attention_jvp", "muon")
_lib = None
_status = {}

STATUS_NAMES = {
    0: "ok",
    1: "timeout: TMA producer waited for a free shared-memory stage",
    2: "timeout: MMA issuer waited for TMA data",
    3: "timeout: epilogue waited for an accumulator",
    4: "timeout: MMA issuer waited for the epilogue",
    5: "timeout: wait on a peer flag",
    6: "bad argument seen on the device",
    7: "timeout inside the attention kernel",
}


class AdanaOptHyper(Structure):
    _fields_ = [
        ("lr", c_float), ("alpha", c_float), ("step", c_float), ("one_minus_kappa", c_float),
        ("clipsnr", c_float), ("eps", c_float), ("gamma3", c_float), ("wd_factor", c_float),
        ("grad_scale", c_float), ("kind", c_int),
        ("beta1", c_float), ("beta2", c_float), ("bc1", c_float), ("bc2", c_float),
        ("beta3", c_float), ("wd_coupled", c_float),
    ]


def _declare(lib):
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    sigs = {
        "adana_gemm_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, P, L, P, L, F, F, I, P, P],
        "adana_gemm_set_mode": [I],
        "adana_gemm_bf16_reduce_scatter": [P, P, P, I, I, I, I, I, I, L, L, L, F, I, P, P],
        "adana_sum_slots_bf16": [P, I, I, I, L, P, L, P, L, P, L, P],
        "adana_p2p_all_to_all_pull": [P, P, I, I, I, L, P, L, P, P, P],
        "adana_p2p_reduce_scatter_bf16": [P, I, L, I, I, L, P, L, P, L, P, L, P],
        "adana_gemm_bf16_gather": [P, P, I, I, P, P, I, I, I, L, L, L, I, I, P, L, P, L, F, I, P, P, P, P],
        "adana_norm_fwd": [P, I, P, P, I, P, P, I, I, F, I, P],
        "adana_norm_bwd": [P, I, P, I, P, P, P, P, I, P, I, I, I, I, P, P],
        "adana_colsum_f32": [P, I, I, P, I, P],
        "adana_qknorm_rope_fwd": [P, L, I, I, I, I, P, P, P, P, P, L, I, I, I, I, F, I, P],
        "adana_qknorm_rope_bwd": [P, P, P, L, I, I, I, I, P, P, P, P, P, P, I, L, I, I, I, I, F, I, I, P],
        "adana_sigmoid_gate_fwd": [P, P, L, I, I, P, L, I, I, P],
        "adana_sigmoid_gate_bwd": [P, P, P, L, I, I, P, P, L, I, I, P],
        "adana_clip_coef": [P, F, F, P, P],
        "adana_p2p_barrier": [P, I, I, I, ctypes.c_uint, ctypes.c_ulonglong, P, P],
        "adana_p2p_reduce_scatter": [P, I, L, L, P, P, P],
        "adana_p2p_publish_f32": [P, I, I, P, P],
        "adana_p2p_signal": [P, I, I, I, ctypes.c_uint, P],
        "adana_p2p_reduce_scatter_flag": [P, I, P, ctypes.c_uint, I, L, L, P, P, ctypes.c_ulonglong, P, P],
        "adana_p2p_all_reduce_flag": [P, I, P, P, ctypes.c_uint, I, L, L, P, ctypes.c_ulonglong, P, P],
        "adana_p2p_push_f32": [P, P, I, L, L, P],
        "adana_clip_coef_multi": [P, I, F, F, P, P],
        "adana_p2p_opt_step_push": [P, P, P, P, P, P, I, L, L, POINTER(AdanaOptHyper), P, P],
        "adana_attn_fwd": [P, P, P, L, I, P, P, I, I, I, I, I, F, P, P],
        "adana_attn_bwd": [P, P, P, L, I, P, P, P, P, P, P, L, I, P, I, I, I, I, I, F, P, P],
        "adana_attn_jvp": [P, P, P, P, P, P, P, P, I, I, I, I, I, F, P, P],
        "adana_embedding_fwd": [P, P, I, P, I, I, I, P],
        "adana_embedding_bwd": [P, P, P, I, I, I, P],
        "adana_ce_fwd_bwd": [P, L, P, I, I, F, F, P, L, P, P, P],
        "adana_ce_fwd_bwd_bf16": [P, L, P, I, I, F, F, P, L, P, P, P],
        "adana_opt_step": [P, P, P, P, P, P, L, POINTER(AdanaOptHyper), P, P, P],
        "adana_sumsq_f32": [P, L, P, P],
        "adana_cast_f32_to_bf16": [P, P, L, P],
        "adana_muon_parts": [],
        "adana_muon_momentum": [P, P, P, P, I, P, F, F, I, P, P],
        "adana_muon_pull": [P, P, I, L, L, L, I, F, P, P, ctypes.c_uint, ctypes.c_ulonglong, P, P],
        "adana_muon_push": [P, P, I, L, L, L, P],
        "adana_muon_apply": [P, P, P, P, P, P, I, P, P, P, I, L, L, P, ctypes.c_uint, I, ctypes.c_ulonglong, P, P],
        "adana_version": [],
    }
    for name, args in sigs.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
    return lib


class _CountingLibrary:
    """Proxy over the ctypes library that counts entry-point calls (each launches one kernel)."""

    def __init__(self, cdll):
        self._cdll = cdll
        self.calls = 0

    def __getattr__(self, name):
        fn = getattr(self._cdll, name)  # AttributeError for a missing symbol keeps hasattr() honest
        if name in ("adana_version", "adana_gemm_set_mode", "adana_muon_parts"):   # host-only entry points launch nothing
            self.__dict__[name] = fn
            return fn

        def counted(*args, _fn=fn):
            self.calls += 1
            return _fn(*args)

        self.__dict__[name] = counted
        return counted


def launch_count() -> int:
    """Number of kernel-library entry points called so far in this process."""
    return 0 if _lib is None else _lib.calls


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    """True when CUDA kernels can run: a GPU is visible and the library loads."""
    if not torch.cuda.is_available():
        return False
    return lib() is not None


def lib():
    """Load (building first if the .so is missing and nvcc exists) and return the library."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        try:
            from adana_b200 import build as _build

            _build.build(debug=DEBUG_BUILD)
        except Exception as e:  # pragma: no cover - depends on toolchain
            if torch.cuda.is_available():
                raise RuntimeError(
                    f"adana_b200: kernel library missing and could not be built: {e}"
                ) from e
            return None
    try:
        _lib = _CountingLibrary(_declare(ctypes.CDLL(str(_LIB_PATH))))
    except OSError as e:
        if torch.cuda.is_available():
            raise RuntimeError(f"adana_b200: cannot load {_LIB_PATH}: {e}") from e
        return None
    return _lib


def has(name: str) -> bool:
    l = lib()
    return l is not None and hasattr(l, name)


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_buffer(device=None) -> torch.Tensor:
    """One int32 status word per device; kernels write a code there when a wait times out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    buf = _status.get(key)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=dev)
        _status[key] = buf
        if DEBUG_BUILD and _lib is not None:
            # checked build: every translation unit reports its range violations into this device's status word
            with torch.cuda.device(dev):
                for unit in _DEBUG_UNITS:
                    check_rc(getattr(_lib._cdll, f"adana_debug_bind_{unit}")(c_void_p(buf.data_ptr())), f"bind {unit}")
    return buf


def check_status(device=None) -> None:
    """Synchronising check of the device status word; raises on a recorded timeout."""
    buf = status_buffer(device)
    code = int(buf[0].item())
    if code != 0:
        buf.zero_()
        raise RuntimeError(f"adana_b200 kernel reported: {STATUS_NAMES.get(code, code)}")


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"adana_b200: {what} failed with code {rc}")
