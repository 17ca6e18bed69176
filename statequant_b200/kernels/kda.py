"""Packed recurrent state for KDA (Kimi Delta Attention) layers: lockstep container and slot layout, stepped by
``sqb_kda_step``.

KDA is gated delta with a decay per KEY channel: S_t = (I - beta k k^T) diag(a_t) S_{t-1} + beta k v^T,
o_t = S_t^T q_t (q, k l2-normalised, q scaled).  The buffer keeps the cumulative log decay per channel: GB is
[H, m, d_k] and GCUR [H, d_k].  Mirrors ``PackedKDAState`` / ``KDASlotLayout`` of the reference
(``src/statequant/kernels/kda.py:208-386``).
"""
from __future__ import annotations

import torch

from .. import _cabi
from .formats import l2norm, pow2
from .layout import KIND_KDA, BlobLayout, set_shape
from .lockstep import LockstepTables


def kda_recurrence(S, q, k, v, g, beta, scale=None):
    """One plain fp32 KDA step on S [BH, d_v, d_k] (value-major, updated in place); returns o [BH, d_v]
    (reference: ``kda.py:44-52``)."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    qn, kn = l2norm(q) * scale, l2norm(k)
    S.mul_(torch.exp(g.float())[:, None, :])
    u = beta.float()[:, None] * (v.float() - torch.einsum('bvk,bk->bv', S, kn))
    S.add_(u[:, :, None] * kn[:, None, :])
    return torch.einsum('bvk,bk->bv', S, qn)


def _common(st, fmt, hv, dk, dv, m, buffer_bits):
    st.state_dtype = torch.bfloat16
    assert min(dk, dv) >= 16 and pow2(dk) == dk and pow2(dv) == dv, f'd_k = {dk}, d_v = {dv}: powers of two from 16 up'
    set_shape(st, fmt, hv, hv, dk, dv, m, buffer_bits, gdn_dims=False, float_group=16)


def _inputs(st, idx, q, k, v, g, beta, out, scale):
    for t in (q, k, v, g):
        assert t.stride(-1) == 1, 'unit inner stride'
    assert q.stride(-2) == st.DK and k.stride(-2) == st.DK and v.stride(-2) == st.DV and g.stride(-2) == st.DK
    assert beta.stride(-1) == 1 and out.stride(-1) == 1 and out.stride(-2) == st.DV and q.dtype == k.dtype
    a = _cabi.KdaInputs()
    a.idx = _cabi.ptr(idx)
    a.q, a.sq, a.k, a.sk, a.qk_dtype = q.data_ptr(), _cabi.row_stride_bytes(q), k.data_ptr(), \
        _cabi.row_stride_bytes(k), _cabi.dtype_code(q)
    a.v, a.sv, a.v_dtype = v.data_ptr(), _cabi.row_stride_bytes(v), _cabi.dtype_code(v)
    a.g, a.sg, a.g_dtype = g.data_ptr(), _cabi.row_stride_bytes(g), _cabi.dtype_code(g)
    a.beta, a.sbeta, a.beta_dtype = beta.data_ptr(), _cabi.row_stride_bytes(beta), _cabi.dtype_code(beta)
    a.out, a.so, a.out_dtype = out.data_ptr(), _cabi.row_stride_bytes(out), _cabi.dtype_code(out)
    a.scale, a.rows = float(scale), out.shape[0]
    return a


class PackedKDAState(LockstepTables):
    """One KDA layer's packed state and decode buffer for B sequences in lockstep.

    S [B, H, d_v, d_k] (or [B*H, d_v, d_k]); ``step(q, k, v, g, beta, scale)`` with q, k raw [B, H, d_k], v
    [.., d_v], g [.., d_k] log decay, beta [B, H]; returns the output buffer [B, H, d_v]."""

    def __init__(self, S, fmt, m=8, hv=None, buffer_bits=8, out_dtype=torch.bfloat16, sbv=None, fbv=None,
                 warps=None):
        S = self._vk(S)
        BH, DV, DK = S.shape
        hv = hv or BH
        assert BH % hv == 0
        _common(self, fmt, hv, DK, DV, m, buffer_bits)
        self.BH, self.B = BH, BH // hv
        self._allocate(S, DK, out_dtype)

    def step(self, q, k, v, g, beta, scale=None):
        Bn, HV, DK, DV = self.B, self.HV, self.DK, self.DV
        q, k = q.reshape(Bn, HV, DK), k.reshape(Bn, HV, DK)
        v, g, beta = v.reshape(Bn, HV, DV), g.reshape(Bn, HV, DK), beta.reshape(Bn, HV)
        a = _inputs(self, None, q, k, v, g, beta, self.O, DK ** -0.5 if scale is None else scale)
        _cabi.check(_cabi.lib().sqb_kda_step(_cabi.C.byref(self._st), _cabi.C.byref(a),
                                             _cabi.current_stream(q.device)), 'sqb_kda_step')
        return self.O


class KDASlotLayout(BlobLayout):
    """The per-slot blob of one KDA layer and the KDA decode step on a batch of slots.

    Fields (16-byte aligned, in this order): GB fp32 [H, m, d_k], GCUR fp32 [H, d_k], NPTR int32 [max(H, 4)], SC,
    KBS / UBS fp16 [H, m] (int8 buffer only), S codes, KB [H, m, d_k], UB [H, m, d_v]."""
    kind = KIND_KDA

    def __init__(self, fmt, hv, dk, dv, m=8, buffer_bits=8, sbv=None, fbv=None, warps=None):
        _common(self, fmt, hv, dk, dv, m, buffer_bits)
        self.fused = True
        self._finish(decay_width=dk, ragged=False)

    _head_words = ('heads', '', 'd_k', 'd_v')

    def step(self, views, idx, q, k, v, g, beta, out, scale=None):
        """One decode token for every batch row b on slot ``idx[b]`` (int32 [rows]; <= 0 = padding).  q, k
        [rows, H, d_k] raw, v [rows, H, d_v], g [rows, H, d_k] log decay, beta [rows, H]; out [rows, H, d_v]."""
        rows = idx.shape[0]
        if rows == 0:
            return out
        assert idx.dtype == torch.int32 and idx.is_contiguous()
        a = _inputs(self, idx, q, k, v, g, beta, out[:rows], self.DK ** -0.5 if scale is None else scale)
        _cabi.check(_cabi.lib().sqb_kda_step(_cabi.C.byref(self._struct(views)), _cabi.C.byref(a),
                                             _cabi.current_stream(q.device)), 'sqb_kda_step')
        return out
