"""Packed recurrent state for Mamba2 / SSD layers: lockstep container and slot layout, stepped by ``sqb_mamba2_step``.

Mamba2 per head h (group g = h // (H / G)), one token:  dt = softplus(dt_raw + dt_bias) clamped to dt_limit,
S <- exp(A_h dt) S + (dt x) B^T,  y = S C + D_h x, with S [head_dim, d_state] = [d_v, d_k] value-major.  In the
delta-buffer picture B is the key (one per group), C the query, u = dt x the buffered value.
Mirrors ``PackedMamba2State`` / ``Mamba2SlotLayout`` of the reference (``src/statequant/kernels/mamba2.py:259-396``).
"""
from __future__ import annotations

import torch

from .. import _cabi
from .layout import KIND_M2, BlobLayout, set_shape
from .lockstep import LockstepTables


def _common(st, fmt, hv, hk, dk, dv, m, buffer_bits):
    st.state_dtype = torch.bfloat16
    set_shape(st, fmt, hv, hk, dk, dv, m, buffer_bits, gdn_dims=False, float_group=16)


def _inputs(st, idx, x, dt, B, Cm, out, A, D, dt_bias, dt_softplus, dt_limit):
    assert x.stride(-1) == 1 and B.stride(-1) == 1 and Cm.stride(-1) == 1 and dt.stride(-1) == 1
    assert x.stride(-2) == st.DV and out.stride(-1) == 1 and out.stride(-2) == st.DV
    assert B.stride(-2) == st.DK and Cm.stride(-2) == st.DK and B.dtype == Cm.dtype
    assert A.is_contiguous() and (D is None or D.is_contiguous()) and (dt_bias is None or dt_bias.is_contiguous())
    clamp = dt_limit is not None and tuple(dt_limit) != (0., float('inf'))
    a = _cabi.Mamba2Inputs()
    a.idx = _cabi.ptr(idx)
    a.x, a.sx, a.x_dtype = x.data_ptr(), _cabi.row_stride_bytes(x), _cabi.dtype_code(x)
    a.dt, a.sdt, a.dt_dtype = dt.data_ptr(), _cabi.row_stride_bytes(dt), _cabi.dtype_code(dt)
    a.B, a.sB, a.C, a.sC, a.bc_dtype = B.data_ptr(), _cabi.row_stride_bytes(B), Cm.data_ptr(), \
        _cabi.row_stride_bytes(Cm), _cabi.dtype_code(B)
    a.A, a.a_dtype = A.data_ptr(), _cabi.dtype_code(A)
    if D is not None:
        a.D, a.d_dtype = D.data_ptr(), _cabi.dtype_code(D)
    if dt_bias is not None:
        a.dt_bias, a.dtb_dtype = dt_bias.data_ptr(), _cabi.dtype_code(dt_bias)
    a.out, a.so, a.out_dtype = out.data_ptr(), _cabi.row_stride_bytes(out), _cabi.dtype_code(out)
    a.dt_softplus, a.dt_clamp = int(bool(dt_softplus)), int(clamp)
    a.dt_min, a.dt_max = (float(dt_limit[0]), float(dt_limit[1])) if clamp else (0., 0.)
    a.rows = out.shape[0]
    return a


def mamba2_recurrence(S, x, dt, B, C, A, D=None, dt_bias=None, dt_softplus=False, dt_limit=None):
    """One plain fp32 Mamba2 step on S [B, H, d_v, d_k] (updated in place); returns y [B, H, d_v] fp32
    (reference: ``mamba2.py:57-70``)."""
    H, G = dt.shape[1], B.shape[1]
    dt = dt.float()
    if dt_bias is not None:
        dt = dt + dt_bias.float()
    if dt_softplus:
        dt = torch.where(dt <= 20., torch.log(1. + torch.exp(dt)), dt)
    if dt_limit is not None and tuple(dt_limit) != (0., float('inf')):
        dt = dt.clamp(dt_limit[0], dt_limit[1])
    g = A.float() * dt
    Bh, Ch = B.float().repeat_interleave(H // G, 1), C.float().repeat_interleave(H // G, 1)
    u = dt[..., None] * x.float()
    S.mul_(torch.exp(g)[..., None, None]).add_(u[..., :, None] * Bh[..., None, :])
    y = torch.einsum('bhvk,bhk->bhv', S, Ch)
    return y if D is None else y + D.float()[:, None] * x.float()


class PackedMamba2State(LockstepTables):
    """One Mamba2 layer's packed state and decode buffer for B sequences in lockstep.

    S [B, H, d_v, d_k] (or [B*H, d_v, d_k]); fmt, m, hv (= H), hk (= G groups), buffer_bits as the slot layout;
    ``sbv, fbv, warps`` are accepted and ignored.  ``step(x, dt, B, C, A, D, dt_bias, dt_softplus, dt_limit)``
    returns the output buffer [B, H, d_v] (the same tensor every step)."""

    def __init__(self, S, fmt, m=8, hv=None, hk=None, buffer_bits=8, out_dtype=torch.bfloat16, sbv=None, fbv=None,
                 warps=None):
        S = self._vk(S)
        BH, DV, DK = S.shape
        hv = hv or BH
        assert BH % hv == 0
        _common(self, fmt, hv, hk or hv, DK, DV, m, buffer_bits)
        self.BH, self.B = BH, BH // hv
        self._allocate(S, 1, out_dtype)

    def step(self, x, dt, B, C, A, D=None, dt_bias=None, dt_softplus=False, dt_limit=None):
        Bn, HV, HK = self.B, self.HV, self.HK
        x = x.reshape(Bn, HV, self.DV)
        dt = dt.reshape(Bn, HV)
        B = B.reshape(Bn, HK, self.DK)
        C = C.reshape(Bn, HK, self.DK)
        a = _inputs(self, None, x, dt, B, C, self.O, A, D, dt_bias, dt_softplus, dt_limit)
        _cabi.check(_cabi.lib().sqb_mamba2_step(_cabi.C.byref(self._st), _cabi.C.byref(a),
                                                _cabi.current_stream(x.device)), 'sqb_mamba2_step')
        return self.O


class Mamba2SlotLayout(BlobLayout):
    """The per-slot blob of one Mamba2 layer (fields as ``SlotLayout``: KB / KBS per group, UB / UBS, GB, GCUR per
    head) and the Mamba2 decode step on a batch of slots.

    fmt, hv (heads on this rank), hk (groups on this rank), dk (d_state), dv (head_dim), m, buffer_bits;
    ``sbv, fbv, warps`` accepted and ignored."""
    kind = KIND_M2

    def __init__(self, fmt, hv, hk, dk, dv, m=8, buffer_bits=8, sbv=None, fbv=None, warps=None):
        _common(self, fmt, hv, hk, dk, dv, m, buffer_bits)
        self.fused = True
        self._finish(ragged=False)

    _head_words = ('heads', 'groups', 'd_state', 'head_dim')

    def step(self, views, idx, x, dt, B, C, out, A, D=None, dt_bias=None, dt_softplus=True,
             dt_limit=(0., float('inf'))):
        """One decode token for every batch row b on slot ``idx[b]`` (int32 [rows]; <= 0 = padding: output zeroed,
        nothing read or written).  x [rows, H, d_v], dt [rows, H] raw, B / C [rows, G, d_k]: any row stride,
        contiguous rows; out [rows, H, d_v]; A [H] (= -exp(A_log)), D, dt_bias [H] or None.  One launch."""
        rows = idx.shape[0]
        if rows == 0:
            return out
        assert idx.dtype == torch.int32 and idx.is_contiguous()
        a = _inputs(self, idx, x, dt, B, C, out[:rows], A, D, dt_bias, dt_softplus, dt_limit)
        _cabi.check(_cabi.lib().sqb_mamba2_step(_cabi.C.byref(self._struct(views)), _cabi.C.byref(a),
                                                _cabi.current_stream(x.device)), 'sqb_mamba2_step')
        return out
