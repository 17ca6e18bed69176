"""Python handle on the CPU oracle (``oracle/sq_oracle.c``).  TEST INFRASTRUCTURE: only tests/, the smoke check
and the benchmark's CPU legs may import this module; the package ``statequant_b200`` never does.

The oracle takes the same argument structs as the C ABI, with host pointers, so a test steps the very same blob
bytes through the CUDA kernels and through the oracle and compares the results byte for byte.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import torch

from statequant_b200 import _cabi
from statequant_b200.kernels import kda as _kda
from statequant_b200.kernels import mamba2 as _m2
from statequant_b200.kernels.slots import _gdn_inputs

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, 'liboracle.so')
_lib = None


def build(force=False):
    srcs = [os.path.join(HERE, f) for f in ('sq_oracle.c', 'sq_oracle_gga.c', 'sq_oracle_conv.c', 'Makefile')]
    srcs.append(os.path.join(HERE, '..', 'include', 'statequant_b200.h'))
    if force or not os.path.exists(LIB) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in srcs):
        subprocess.run(['make', '-C', HERE, '-B', 'liboracle.so'], check=True, capture_output=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        L = C.CDLL(LIB)
        for n in ('sqo_gdn_step', 'sqo_mamba2_step', 'sqo_kda_step'):
            getattr(L, n).restype = C.c_int
            getattr(L, n).argtypes = [C.c_void_p, C.c_void_p]
        L.sqo_num_threads.restype = C.c_int
        L.sqo_conv1d_update.restype = C.c_int
        L.sqo_conv1d_update.argtypes = [C.c_void_p]
        L.sqo_gga_step.restype = L.sqo_gga_store.restype = L.sqo_gga_load.restype = C.c_int
        _lib = L
    return _lib


def _cpu(*ts):
    for t in ts:
        assert t is None or t.device.type == 'cpu', 'the oracle works on host memory'


def num_threads():
    return int(lib().sqo_num_threads())


def set_num_threads(n):
    """Threads of the oracle's parallel loops from now on (overrides OMP_NUM_THREADS)."""
    lib().sqo_set_num_threads(int(n))


def pack_vk(x, bits, axis_k, group):
    """fp32 [n, dv, dk] -> (codes, scales) with the oracle's packer."""
    x = x.float().contiguous()
    n, dv, dk = x.shape
    if bits == 4:
        codes = torch.empty(n, dv, dk // 2, dtype=torch.uint8)
    elif bits == 8:
        codes = torch.empty(n, dv, dk, dtype=torch.int8)
    else:
        codes = torch.empty(n, dv, dk, dtype=torch.bfloat16 if bits == 16 else torch.float32)
    ns = (dv * -(-dk // group) if axis_k else (dv // group) * dk) if bits <= 8 else 1
    scales = torch.ones(n, ns, dtype=torch.float16)
    lib().sqo_pack_vk(C.c_void_p(x.data_ptr()), C.c_int64(n), dv, dk, bits, int(axis_k), group,
                      C.c_void_p(codes.data_ptr()), C.c_void_p(scales.data_ptr()))
    if bits <= 8:
        scales = scales.view(n, dv, -1) if axis_k else scales.view(n, dv // group, dk)
    return codes, scales


def unpack_vk(codes, scales, bits, axis_k, group, dk):
    n, dv = codes.shape[:2]
    x = torch.empty(n, dv, dk, dtype=torch.float32)
    codes, scales = codes.contiguous(), scales.contiguous()
    lib().sqo_unpack_vk(C.c_void_p(codes.data_ptr()), C.c_void_p(scales.data_ptr()), C.c_int64(n), dv, dk, bits,
                        int(axis_k), group, C.c_void_p(x.data_ptr()))
    return x


def gdn_step(lay, views, idx, q, k, v, out, scale, *, g=None, beta=None, gate=None, per_key_head=True):
    """``SlotLayout.step`` on host memory through the oracle."""
    _cpu(views['S'], idx, q, k, v, out)
    a = _gdn_inputs(idx, q, k, v, out, scale, g, beta, gate, per_key_head)
    st = lay._struct(views)
    rc = lib().sqo_gdn_step(C.byref(st), C.byref(a))
    assert rc == 0
    return out


def mamba2_step(lay, views, idx, x, dt, B, Cm, out, A, D=None, dt_bias=None, dt_softplus=True,
                dt_limit=(0., float('inf'))):
    _cpu(views['S'], idx, x, dt, B, Cm, out)
    a = _m2._inputs(lay, idx, x, dt, B, Cm, out, A, D, dt_bias, dt_softplus, dt_limit)
    rc = lib().sqo_mamba2_step(C.byref(lay._struct(views)), C.byref(a))
    assert rc == 0
    return out


def kda_step(lay, views, idx, q, k, v, g, beta, out, scale=None):
    _cpu(views['S'], idx, q, k, v, g, beta, out)
    a = _kda._inputs(lay, idx, q, k, v, g, beta, out, lay.DK ** -0.5 if scale is None else scale)
    rc = lib().sqo_kda_step(C.byref(lay._struct(views)), C.byref(a))
    assert rc == 0
    return out


def slot_read(lay, views, slots):
    """``layout.read`` through the oracle: fp32 [P, HV, DV, DK]."""
    slots = slots.to(torch.int64).contiguous()
    P = slots.shape[0]
    out = torch.empty(P, lay.HV, lay.DV, lay.DK, dtype=torch.float32)
    rc = lib().sqo_slot_read(C.byref(lay._struct(views)), int(lay.kind), C.c_void_p(slots.data_ptr()), C.c_int64(P),
                             C.c_void_p(out.data_ptr()))
    assert rc == 0
    return out


def slot_write(lay, views, slots, S):
    slots = slots.to(torch.int64).contiguous()
    S = S.float().contiguous()
    rc = lib().sqo_slot_write(C.byref(lay._struct(views)), int(lay.kind), C.c_void_p(slots.data_ptr()),
                              C.c_int64(slots.shape[0]), C.c_void_p(S.data_ptr()))
    assert rc == 0


# ---- GGA / STEP ---------------------------------------------------------------------------------------------------
def stepquant_fit(x, bits, w, group=32):
    """step_quant.fit through the oracle: x [B, H, dk, dv] fp32 (host)."""
    x = x.float().contiguous()
    y = torch.empty_like(x)
    bits = bits.to(torch.int32).contiguous()
    w = w.float().contiguous()
    B, H, dk, dv = x.shape
    lib().sqo_stepquant_fit(C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), C.c_void_p(bits.data_ptr()),
                            C.c_void_p(w.data_ptr()), C.c_int64(B), H, dk, dv, group)
    return y


def gga_step(pk, views, idx, q, k, v, out, scale, gate, layer):
    """``GGAPacked.step`` (step + counter advance) on host memory through the oracle."""
    _cpu(views['blob'], idx, q, k, v, out)
    a = _gdn_inputs(idx, q, k, v, out, scale, None, None, gate, True)
    rc = lib().sqo_gga_step(C.byref(pk._struct(views, layer)), C.byref(a))
    assert rc == 0
    return out


def gga_store(pk, views, idx, S, layer):
    """``GGAPacked.write``: S value-major [P, HV, dv, dk]."""
    idx32 = idx.to(torch.int32).contiguous()
    X = S.float().transpose(-1, -2).contiguous()
    rc = lib().sqo_gga_store(C.byref(pk._struct(views, layer)), C.c_void_p(idx32.data_ptr()), C.c_int64(idx32.shape[0]),
                             C.c_void_p(X.data_ptr()))
    assert rc == 0


def gga_load(pk, views, idx, layer):
    """``GGAPacked.stored``: canonical fp32 [P, HV, dk, dv]."""
    idx32 = idx.to(torch.int32).contiguous()
    Y = torch.empty(idx32.shape[0], pk.HV, pk.DK, pk.DV)
    rc = lib().sqo_gga_load(C.byref(pk._struct(views, layer)), C.c_void_p(idx32.data_ptr()), C.c_int64(idx32.shape[0]),
                            C.c_void_p(Y.data_ptr()))
    assert rc == 0
    return Y


def conv1d_update(x, conv_state, weight, bias=None, activation=None, conv_state_indices=None, null_block_id=0):
    """The oracle's causal conv update on host tensors, in place on x and conv_state (arguments as
    ``statequant_b200.kernels.conv.causal_conv1d_update``); returns x."""
    _cpu(x, conv_state, weight, bias, conv_state_indices)
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype == conv_state.dtype
    rows, dim = x.shape
    es, ws = x.element_size(), weight.element_size()
    idx = conv_state_indices
    if idx is not None:
        idx = idx.to(torch.int32).contiguous()
    a = _cabi.ConvUpdate(
        x=x.data_ptr(), sx=x.stride(0) * es, out=x.data_ptr(), so=x.stride(0) * es,
        state=conv_state.data_ptr(), s_line=conv_state.stride(0) * es, s_dim=conv_state.stride(1) * es,
        s_tok=conv_state.stride(2) * es, w=weight.data_ptr(), sw_dim=weight.stride(0) * ws,
        sw_tap=weight.stride(1) * ws, bias=_cabi.ptr(bias), idx=_cabi.ptr(idx), rows=rows, dim=dim,
        width=weight.size(1), state_len=conv_state.size(2), x_dtype=_cabi.dtype_code(x),
        w_dtype=_cabi.dtype_code(weight), silu=int(bool(activation)),
        null_line=-1 if null_block_id is None else int(null_block_id))
    rc = lib().sqo_conv1d_update(C.byref(a))
    assert rc == 0, f'sqo_conv1d_update: {rc}'
    return x
