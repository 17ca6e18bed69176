"""Lockstep packed Gated DeltaNet state (all sequences at the same buffer position) and the format helpers.

``PackedGDNState`` mirrors the reference container of that name (``src/statequant/kernels/fold.py:280-424``): the
same constructor, attributes (``codes scales KB UB KBS UBS GB GCUR NPTR O``), ``step``, ``load``, ``dequantize``,
``n`` and ``stored_bytes``.  Every tensor is allocated once and written in place, so ``step`` can be captured in a
CUDA graph.  The step is one launch of the sm_100a kernel through ``sqb_gdn_step`` with the identity slot map.
"""
from __future__ import annotations

import torch

from .. import _cabi
from .formats import (check_dims, l2norm, pack, pack_vk, packed_format, pow2, state_bits, unpack,  # noqa: F401
                      unpack_vk)
from .layout import state_struct
from .slots import _gdn_inputs


def _flat3(S):
    return S.float().reshape(-1, S.shape[-2], S.shape[-1]).contiguous()


class PackedGDNState:
    """One layer's packed recurrent state and decode buffer for B sequences in lockstep.

    S            [BH, d_k, d_v] (or [B, H, d_k, d_v]) float state to start from
    fmt          ``Quantizer(bits in {4, 8}, axis in {'k', 'v'}, group)`` or 'bf16'; scales are stored fp16
    m            buffer length (power of two); hv, hk value / key heads per sequence; buffer_bits 8 or 16
    out_dtype    dtype of the output
    block_v, warps, fused, fused_warps   accepted and ignored (tuning knobs of the reference's Triton path)

    ``step(q, k, v, g, beta, scale)``: q, k raw [BH, d_k] or per key head [B * hk, d_k]; v [BH, d_v]; g, beta [BH].
    Returns the output buffer [BH, d_v] (the same tensor every step).
    """

    def __init__(self, S, fmt, m=8, hv=None, hk=None, buffer_bits=8, out_dtype=torch.bfloat16,
                 block_v=None, warps=None, fused=None, fused_warps=None):
        S = _flat3(S)
        BH, DK, DV = S.shape
        dev = S.device
        self.BH, self.DK, self.DV, self.m = BH, DK, DV, m
        self.fmt = packed_format(fmt)
        self.bits = state_bits(self.fmt)
        self.HV = hv or BH
        self.HK = hk or self.HV
        assert self.HV % self.HK == 0 and BH % self.HV == 0, (BH, self.HV, self.HK)
        self.gqa, self.B = self.HV // self.HK, BH // self.HV
        assert m >= 1 and m & (m - 1) == 0, 'm must be a power of two'
        check_dims(self.fmt, DK, DV)
        assert buffer_bits in (8, 16)
        self.buffer_bits, self.qbuf = buffer_bits, buffer_bits == 8
        self.axk = self.fmt is not None and self.fmt.axis == 'k'
        self.group = self.fmt.group if self.fmt is not None else 32
        self.fused = True
        codes, scales = pack(S, self.fmt)
        self.codes, self.scales = codes.clone(), scales.clone()
        bdt = torch.int8 if self.qbuf else torch.bfloat16
        B, HK, HV = self.B, self.HK, self.HV
        self.KB = torch.zeros(B * HK, m, DK, device=dev, dtype=bdt)
        self.UB = torch.zeros(BH, m, DV, device=dev, dtype=bdt)
        self.KBS = torch.zeros(B * HK, m, device=dev, dtype=torch.float16)
        self.UBS = torch.zeros(BH, m, device=dev, dtype=torch.float16)
        self.GB = torch.zeros(BH, m, device=dev, dtype=torch.float32)
        self.GCUR = torch.zeros(BH, device=dev, dtype=torch.float32)
        self.NPTR = torch.zeros(B, HV, device=dev, dtype=torch.int32)
        self.O = torch.zeros(BH, DV, device=dev, dtype=out_dtype)
        tabs = dict(S=self.codes, SC=self.scales if self.fmt is not None else None, KB=self.KB, KBS=self.KBS,
                    UB=self.UB, UBS=self.UBS, GB=self.GB, GCUR=self.GCUR, NPTR=self.NPTR)
        per_seq = dict(S=HV * self.codes[0].numel() * self.codes.element_size(),
                       SC=HV * self.scales[0].numel() * 2 if self.fmt is not None else 0,
                       KB=HK * m * DK * self.KB.element_size(), KBS=HK * m * 2,
                       UB=HV * m * DV * self.UB.element_size(), UBS=HV * m * 2, GB=HV * m * 4, GCUR=HV * 4,
                       NPTR=HV * 4)
        self._st = state_struct(tabs, per_seq, bits=self.bits, axis_k=self.axk, group=self.group,
                                buffer_bits=buffer_bits, m=m, hv=HV, hk=HK, dk=DK, dv=DV)

    @torch.no_grad()
    def load(self, S):
        """Replace the state (in place) and empty the buffer."""
        c, sc = pack(_flat3(S), self.fmt)
        self.codes.copy_(c)
        self.scales.copy_(sc)
        for t in (self.KB, self.UB, self.KBS, self.UBS, self.GB, self.GCUR, self.NPTR):
            t.zero_()

    def dequantize(self):
        """The stored state S_0 (without the buffered tokens) as [BH, d_k, d_v] fp32."""
        return unpack(self.codes, self.scales, self.fmt, self.DK)

    @property
    def n(self):
        return int(self.NPTR.reshape(-1)[0])

    def stored_bytes(self):
        """Resident bytes: state payload + scales, the buffer, the decays."""
        nb = lambda t: t.numel() * t.element_size()          # noqa: E731
        per = dict(state=nb(self.codes) + (nb(self.scales) if self.fmt is not None else 0),
                   buffer=nb(self.KB) + nb(self.UB) + ((nb(self.KBS) + nb(self.UBS)) if self.qbuf else 0),
                   decay=nb(self.GB) + nb(self.GCUR) + nb(self.NPTR))
        per['total'] = sum(per.values())
        return per

    def step(self, q, k, v, g, beta, scale):
        B, HV, HK, DK, DV = self.B, self.HV, self.HK, self.DK, self.DV
        per_key = q.shape[0] != self.BH
        if per_key:
            assert q.shape[0] == B * HK and k.shape[0] == B * HK
        for t in (q, k, v, g, beta):
            assert t.is_contiguous()
        hq = HK if per_key else HV
        a = _gdn_inputs(None, q.view(B, hq, DK), k.view(B, hq, DK), v.view(B, HV, DV), self.O.view(B, HV, DV), scale,
                        g.view(B, HV), beta.view(B, HV), None, per_key)
        _cabi.check(_cabi.lib().sqb_gdn_step(_cabi.C.byref(self._st), _cabi.C.byref(a),
                                             _cabi.current_stream(q.device)), 'sqb_gdn_step')
        return self.O
