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
from .layout import set_shape
from .lockstep import LockstepTables
from .slots import _gdn_inputs


class PackedGDNState(LockstepTables):
    """One layer's packed recurrent state and decode buffer for B sequences in lockstep.

    S            [BH, d_k, d_v] (or [B, H, d_k, d_v]) float state to start from (key-major, as the reference hands it)
    fmt          ``Quantizer(bits in {4, 8}, axis in {'k', 'v'}, group)`` or 'bf16'; scales are stored fp16
    m            buffer length (power of two); hv, hk value / key heads per sequence; buffer_bits 8 or 16
    out_dtype    dtype of the output
    block_v, warps, fused, fused_warps   accepted and ignored (tuning knobs of the reference's Triton path)

    ``step(q, k, v, g, beta, scale)``: q, k raw [BH, d_k] or per key head [B * hk, d_k]; v [BH, d_v]; g, beta [BH].
    Returns the output buffer [BH, d_v] (the same tensor every step).
    """
    _key_major_io = True

    def __init__(self, S, fmt, m=8, hv=None, hk=None, buffer_bits=8, out_dtype=torch.bfloat16,
                 block_v=None, warps=None, fused=None, fused_warps=None):
        S = self._vk(S)
        BH, DV, DK = S.shape
        hv = hv or BH
        assert BH % hv == 0, f'{BH} state heads are not whole sequences of {hv}'
        set_shape(self, fmt, hv, hk or hv, DK, DV, m, buffer_bits, gdn_dims=True, float_group=32)
        self.BH, self.B = BH, BH // hv
        self.fused = True
        self._allocate(S, 1, out_dtype)
        self.O = self.O.view(BH, DV)
        for k in ('GB', 'GCUR'):                         # one row per (sequence, head), as the reference shapes them
            self.T[k] = self.T[k].view(BH, *self.T[k].shape[1:])

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
