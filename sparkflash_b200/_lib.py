"""ctypes access to the two native libraries.

``host()`` returns ``libsfb_host.so`` (built on demand with g++ when missing); ``cuda()`` returns
``libsfb_cuda.so`` and refuses to fall back: when a CUDA device is present and the library is
missing or fails to load, the error is raised to the caller.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_ROOT = Path(__file__).resolve().parent
_host = None
_cuda = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_i64 = ctypes.c_int64
c_f32 = ctypes.c_float
c_u8 = ctypes.c_uint8
c_u64 = ctypes.c_uint64


def _ensure_built() -> None:
    h = _ROOT / "lib" / "libsfb_host.so"
    c = _ROOT / "lib" / "libsfb_cuda.so"
    if h.exists() and c.exists() and not os.environ.get("SFB_REBUILD"):
        return
    from . import _build
    _build.build()


def host() -> ctypes.CDLL:
    global _host
    if _host is None:
        _ensure_built()
        _host = ctypes.CDLL(str(_ROOT / "lib" / "libsfb_host.so"))
        _declare_host(_host)
    return _host


def cuda() -> ctypes.CDLL:
    global _cuda
    if _cuda is None:
        _ensure_built()
        _cuda = ctypes.CDLL(str(_ROOT / "lib" / "libsfb_cuda.so"))
    return _cuda


def _declare_host(L: ctypes.CDLL) -> None:
    L.sfb_f32_to_e4m3.argtypes = [c_f32]; L.sfb_f32_to_e4m3.restype = c_u8
    L.sfb_e4m3_to_f32.argtypes = [c_u8]; L.sfb_e4m3_to_f32.restype = c_f32
    L.sfb_f32_to_e2m1.argtypes = [c_f32]; L.sfb_f32_to_e2m1.restype = c_u8
    L.sfb_e2m1_to_f32.argtypes = [c_u8]; L.sfb_e2m1_to_f32.restype = c_f32
    L.sfb_ue8m0_to_f32.argtypes = [c_u8]; L.sfb_ue8m0_to_f32.restype = c_f32
    L.sfb_ue8m0_ceil.argtypes = [c_f32]; L.sfb_ue8m0_ceil.restype = c_u8
    L.sfb_act_scale_code_fp8.argtypes = [c_f32]; L.sfb_act_scale_code_fp8.restype = c_u8
    L.sfb_act_scale_code_fp4.argtypes = [c_f32]; L.sfb_act_scale_code_fp4.restype = c_u8
    L.sfb_f32_to_bf16.argtypes = [c_f32]; L.sfb_f32_to_bf16.restype = ctypes.c_uint16
    L.sfb_sf_offset.argtypes = [c_i64, c_i64, c_i64]; L.sfb_sf_offset.restype = c_i64
    L.sfb_sf_bytes.argtypes = [c_i64, c_i64]; L.sfb_sf_bytes.restype = c_i64
    for name in ("sfb_act_quant_fp8", "sfb_act_quant_fp4", "sfb_kv_quant_fp4"):
        getattr(L, name).argtypes = [c_void_p, c_i64, c_i64, c_void_p, c_void_p]
        getattr(L, name).restype = None
    for name in ("sfb_act_dequant_fp8", "sfb_kv_dequant_fp4"):
        getattr(L, name).argtypes = [c_void_p, c_void_p, c_i64, c_i64, c_void_p]
        getattr(L, name).restype = None
    for name in ("sfb_weight_quant_fp8_block32", "sfb_weight_quant_fp4_row32"):
        getattr(L, name).argtypes = [c_void_p, c_i64, c_i64, c_void_p, c_void_p]
        getattr(L, name).restype = None
    L.sfb_scales_to_prepared.argtypes = [c_void_p, c_i64, c_i64, c_i64, c_void_p]
    L.sfb_scales_to_prepared.restype = None
