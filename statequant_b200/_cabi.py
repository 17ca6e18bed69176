"""ctypes binding of the C ABI declared in ``include/statequant_b200.h``.

The shared library is built in-tree by ``statequant_b200.build`` (nvcc, sm_100a).  There is no fallback: if the
library is missing or a kernel launch is refused, the call raises.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'lib', 'libstatequant_b200.so')
ABI_VERSION = 1

SQB_F32, SQB_BF16, SQB_F16 = 0, 1, 2
_DT = {torch.float32: SQB_F32, torch.bfloat16: SQB_BF16, torch.float16: SQB_F16}

vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int32, C.c_float


class State(C.Structure):
    """``sqb_state_t``"""
    _fields_ = [('S', vp), ('sS', i64), ('SC', vp), ('sSC', i64), ('KB', vp), ('sKB', i64), ('KBS', vp),
                ('sKBS', i64), ('UB', vp), ('sUB', i64), ('UBS', vp), ('sUBS', i64), ('GB', vp), ('sGB', i64),
                ('GCUR', vp), ('sGC', i64), ('NPTR', vp), ('sN', i64),
                ('bits', i32), ('axis_k', i32), ('group', i32), ('buffer_bits', i32), ('m', i32),
                ('hv', i32), ('hk', i32), ('dk', i32), ('dv', i32), ('reserved', i32)]


class GdnInputs(C.Structure):
    """``sqb_gdn_inputs_t``"""
    _fields_ = [('idx', vp), ('q', vp), ('sq', i64), ('k', vp), ('sk', i64), ('v', vp), ('sv', i64),
                ('g', vp), ('sg', i64), ('beta', vp), ('sbeta', i64), ('a', vp), ('sa', i64), ('b', vp), ('sb', i64),
                ('A_log', vp), ('dt_bias', vp), ('out', vp), ('so', i64),
                ('scale', f32), ('rows', i32), ('qk_per_key_head', i32), ('gate', i32),
                ('qk_dtype', i32), ('v_dtype', i32), ('gb_dtype', i32), ('ab_dtype', i32), ('alog_dtype', i32),
                ('dtb_dtype', i32), ('out_dtype', i32), ('reserved', i32)]


class Mamba2Inputs(C.Structure):
    """``sqb_mamba2_inputs_t``"""
    _fields_ = [('idx', vp), ('x', vp), ('sx', i64), ('dt', vp), ('sdt', i64), ('B', vp), ('sB', i64),
                ('C', vp), ('sC', i64), ('A', vp), ('D', vp), ('dt_bias', vp), ('out', vp), ('so', i64),
                ('dt_min', f32), ('dt_max', f32), ('rows', i32), ('dt_softplus', i32), ('dt_clamp', i32),
                ('x_dtype', i32), ('dt_dtype', i32), ('bc_dtype', i32), ('a_dtype', i32), ('d_dtype', i32),
                ('dtb_dtype', i32), ('out_dtype', i32)]


class KdaInputs(C.Structure):
    """``sqb_kda_inputs_t``"""
    _fields_ = [('idx', vp), ('q', vp), ('sq', i64), ('k', vp), ('sk', i64), ('v', vp), ('sv', i64),
                ('g', vp), ('sg', i64), ('beta', vp), ('sbeta', i64), ('out', vp), ('so', i64),
                ('scale', f32), ('rows', i32), ('qk_dtype', i32), ('v_dtype', i32), ('g_dtype', i32),
                ('beta_dtype', i32), ('out_dtype', i32), ('reserved', i32)]


class ConvUpdate(C.Structure):
    """``sqb_conv_update_t``"""
    _fields_ = [('x', vp), ('sx', i64), ('out', vp), ('so', i64), ('state', vp), ('s_line', i64), ('s_dim', i64),
                ('s_tok', i64), ('w', vp), ('sw_dim', i64), ('sw_tap', i64), ('bias', vp), ('idx', vp),
                ('rows', i32), ('dim', i32), ('width', i32), ('state_len', i32), ('x_dtype', i32), ('w_dtype', i32),
                ('silu', i32), ('null_line', i32)]


def dtype_code(t):
    """SQB_* element type of a tensor (fp32, bf16 or fp16)."""
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f'unsupported activation dtype {t.dtype}; use fp32, bf16 or fp16') from None


def ptr(t):
    return None if t is None else t.data_ptr()


def row_stride_bytes(t):
    """Bytes between consecutive batch rows of a [rows, ...] tensor."""
    return t.stride(0) * t.element_size()


_lib = None


def lib():
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f'{LIB_PATH} is missing: build it with `python -m statequant_b200.build` '
                               '(needs nvcc; there is no CPU or Triton fallback)')
        L = C.CDLL(LIB_PATH)
        L.sqb_last_error.restype = C.c_char_p
        L.sqb_abi_version.restype = C.c_int
        L.sqb_launch_count.restype = C.c_int64
        for name in ('sqb_gdn_step', 'sqb_mamba2_step', 'sqb_kda_step', 'sqb_gga_step'):
            f = getattr(L, name)
            f.restype = C.c_int
            f.argtypes = [vp, vp, vp]
        L.sqb_gga_store.restype = L.sqb_gga_load.restype = L.sqb_stepquant_fit.restype = C.c_int
        L.sqb_gga_store.argtypes = [vp, vp, i64, vp, vp]
        L.sqb_gga_load.argtypes = [vp, vp, i64, vp, vp]
        L.sqb_stepquant_fit.argtypes = [vp, vp, vp, vp, i64, i32, i32, i32, i32, vp]
        L.sqb_slot_read.restype = L.sqb_slot_write.restype = C.c_int
        L.sqb_slot_read.argtypes = [vp, i32, vp, i32, vp, vp]
        L.sqb_slot_write.argtypes = [vp, i32, vp, i32, vp, vp]
        L.sqb_conv1d_update.restype = C.c_int
        L.sqb_conv1d_update.argtypes = [vp, vp]
        L.sqb_set_option.restype = C.c_int
        L.sqb_set_option.argtypes = [C.c_char_p, C.c_int]
        L.sqb_device_status.restype = C.c_int
        L.sqb_device_status.argtypes = [C.POINTER(C.c_int)]
        if L.sqb_abi_version() != ABI_VERSION:
            raise RuntimeError(f'{LIB_PATH} has ABI {L.sqb_abi_version()}, this package expects {ABI_VERSION}: rebuild')
        _lib = L
    return _lib


def check(rc, what):
    if rc != 0:
        raise RuntimeError(f'{what} failed ({rc}): {lib().sqb_last_error().decode()}')


def current_stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def launch_count():
    return int(lib().sqb_launch_count())


def set_option(name, value):
    check(lib().sqb_set_option(name.encode(), int(value)), 'sqb_set_option')


def device_status():
    """Number of CTAs whose bounded wait for a bulk copy ran out (0 in a healthy run); synchronises the device."""
    n = C.c_int(0)
    check(lib().sqb_device_status(C.byref(n)), 'sqb_device_status')
    return n.value
