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
from .formats import l2norm, pack_vk, packed_format, state_bits, unpack_vk
from .layout import KIND_KDA, BlobLayout, state_struct


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
    st.fmt = packed_format(fmt)
    st.bits = state_bits(st.fmt)
    st.state_dtype = torch.bfloat16
    st.HV, st.HK, st.DK, st.DV, st.m = hv, hv, dk, dv, m
    assert dk >= 16 and dk & (dk - 1) == 0 and dv >= 16 and dv & (dv - 1) == 0, (dk, dv)
    assert m >= 1 and m & (m - 1) == 0 and m <= 32, 'm must be a power of two <= 32'
    assert buffer_bits in (8, 16), buffer_bits
    if st.fmt is not None:
        g = st.fmt.group
        assert g >= 2 and g & (g - 1) == 0, f'group {g} must be a power of two'
        assert (dk if st.fmt.axis == 'k' else dv) % g == 0, f'group {g} must divide d_{st.fmt.axis} ({dk}, {dv})'
    st.gqa = 1
    st.buffer_bits, st.qbuf = buffer_bits, buffer_bits == 8
    st.axk = st.fmt is not None and st.fmt.axis == 'k'
    st.group = st.fmt.group if st.fmt is not None else 16


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


class PackedKDAState:
    """One KDA layer's packed state and decode buffer for B sequences in lockstep.

    S [B, H, d_v, d_k] (or [B*H, d_v, d_k]); ``step(q, k, v, g, beta, scale)`` with q, k raw [B, H, d_k], v
    [.., d_v], g [.., d_k] log decay, beta [B, H]; returns the output buffer [B, H, d_v]."""

    def __init__(self, S, fmt, m=8, hv=None, buffer_bits=8, out_dtype=torch.bfloat16, sbv=None, fbv=None,
                 warps=None):
        S = S.float().reshape(-1, S.shape[-2], S.shape[-1])
        BH, DV, DK = S.shape
        hv = hv or BH
        assert BH % hv == 0
        _common(self, fmt, hv, DK, DV, m, buffer_bits)
        self.BH, self.B = BH, BH // hv
        dev = S.device
        c, s = pack_vk(S, self.fmt)
        bdt = torch.int8 if self.qbuf else torch.bfloat16
        self.T = dict(S=c.clone(), SC=s.clone(),
                      KB=torch.zeros(BH, m, DK, device=dev, dtype=bdt),
                      UB=torch.zeros(BH, m, DV, device=dev, dtype=bdt),
                      KBS=torch.zeros(BH, m, device=dev, dtype=torch.float16),
                      UBS=torch.zeros(BH, m, device=dev, dtype=torch.float16),
                      GB=torch.zeros(BH, m, DK, device=dev), GCUR=torch.zeros(BH, DK, device=dev),
                      NPTR=torch.zeros(self.B, hv, device=dev, dtype=torch.int32))
        self.O = torch.zeros(self.B, hv, DV, device=dev, dtype=out_dtype)
        T = self.T
        per_seq = dict(S=hv * T['S'][0].numel() * T['S'].element_size(),
                       SC=hv * T['SC'][0].numel() * 2 if self.fmt is not None else 0,
                       KB=hv * m * DK * T['KB'].element_size(), KBS=hv * m * 2,
                       UB=hv * m * DV * T['UB'].element_size(), UBS=hv * m * 2, GB=hv * m * DK * 4,
                       GCUR=hv * DK * 4, NPTR=hv * 4)
        tabs = dict(T)
        if self.fmt is None:
            tabs['SC'] = None
        self._st = state_struct(tabs, per_seq, bits=self.bits, axis_k=self.axk, group=self.group,
                                buffer_bits=buffer_bits, m=m, hv=hv, hk=hv, dk=DK, dv=DV)

    def __getattr__(self, name):
        T = self.__dict__.get('T')
        if T is not None and name in T:
            return T[name]
        raise AttributeError(name)

    @property
    def codes(self):
        return self.T['S']

    @property
    def scales(self):
        return self.T['SC']

    @property
    def n(self):
        return int(self.T['NPTR'].reshape(-1)[0])

    @torch.no_grad()
    def load(self, S):
        c, s = pack_vk(S.float().reshape(self.BH, self.DV, self.DK), self.fmt)
        self.T['S'].copy_(c)
        self.T['SC'].copy_(s)
        for k in ('KB', 'UB', 'KBS', 'UBS', 'GB', 'GCUR', 'NPTR'):
            self.T[k].zero_()

    def dequantize(self):
        return unpack_vk(self.T['S'], self.T['SC'], self.fmt, self.DK)

    def stored_bytes(self):
        nb = lambda t: t.numel() * t.element_size()          # noqa: E731
        T = self.T
        per = dict(state=nb(T['S']) + (nb(T['SC']) if self.fmt is not None else 0),
                   buffer=nb(T['KB']) + nb(T['UB']) + ((nb(T['KBS']) + nb(T['UBS'])) if self.qbuf else 0),
                   decay=nb(T['GB']) + nb(T['GCUR']) + nb(T['NPTR']))
        per['total'] = sum(per.values())
        return per

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

    def __repr__(self):
        f = 'bf16' if self.fmt is None else f'int{self.bits}-{self.fmt.axis}-g{self.group}'
        return (f'KDASlotLayout({f}, heads={self.HV}, d_k={self.DK}, d_v={self.DV}, m={self.m}, '
                f'buffer_bits={self.buffer_bits}, {self.nbytes} B/slot)')

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
