"""What the three lockstep containers (``PackedGDNState``, ``PackedMamba2State``, ``PackedKDAState``) share: B sequences
that sit at the same buffer position, every table a tensor of its own, allocated once and written in place (so that a
step can be captured in a CUDA graph).

The tables are kept in one dict keyed by the slot layouts' field names (S, SC, KB, KBS, UB, UBS, GB, GCUR, NPTR); the
reference's attribute names (``codes``, ``scales``, ``KB`` ...) resolve to it.  The C-ABI state struct is filled from
the tensors themselves: the stride between two sequences of a table is the table's byte size divided by B.
"""
from __future__ import annotations

import torch

from .formats import pack_vk, unpack_vk
from .layout import state_struct

_BUFFER = ('KB', 'UB', 'KBS', 'UBS', 'GB', 'GCUR', 'NPTR')
_ALIAS = {'codes': 'S', 'scales': 'SC'}


def _nbytes(t):
    return t.numel() * t.element_size()


class LockstepTables:
    """Owner of the per-table tensors of a lockstep container.  Subclasses set the shape attributes (B, HV, HK, DK, DV,
    m, fmt, bits, axk, group, buffer_bits, qbuf) and call ``_allocate``."""

    #: state is handed over and handed back value-major [.., d_v, d_k] unless a subclass says otherwise
    _key_major_io = False

    def _allocate(self, S_vk, decay_width, out_dtype):
        """S_vk fp32 [B * HV, d_v, d_k]: the states to start from.  decay_width: floats of running log decay per head
        (1, or d_k for decays per key channel)."""
        dev, B, HV, HK, DK, DV, m = S_vk.device, self.B, self.HV, self.HK, self.DK, self.DV, self.m
        codes, scales = pack_vk(S_vk, self.fmt)
        buf = torch.int8 if self.qbuf else torch.bfloat16
        z = lambda *shape, dtype=torch.float32: torch.zeros(*shape, device=dev, dtype=dtype)      # noqa: E731
        gshape = (m, decay_width) if decay_width > 1 else (m,)
        cshape = (decay_width,) if decay_width > 1 else ()
        self.T = {'S': codes.clone(), 'SC': scales.clone(),
                  'KB': z(B * HK, m, DK, dtype=buf), 'KBS': z(B * HK, m, dtype=torch.float16),
                  'UB': z(B * HV, m, DV, dtype=buf), 'UBS': z(B * HV, m, dtype=torch.float16),
                  'GB': z(B * HV, *gshape), 'GCUR': z(B * HV, *cshape), 'NPTR': z(B, HV, dtype=torch.int32)}
        self.O = z(B, HV, DV, dtype=out_dtype)
        tabs = dict(self.T)
        if self.fmt is None:
            tabs['SC'] = None                                 # float states carry no scales
        strides = {k: _nbytes(t) // B for k, t in self.T.items()}
        self._st = state_struct(tabs, strides, bits=self.bits, axis_k=self.axk, group=self.group,
                                buffer_bits=self.buffer_bits, m=m, hv=HV, hk=HK, dk=DK, dv=DV)

    # the reference's attribute names
    def __getattr__(self, name):
        T = self.__dict__.get('T')
        key = _ALIAS.get(name, name)
        if T is not None and key in T:
            return T[key]
        raise AttributeError(name)

    @property
    def n(self):
        """Buffer entries in use (the same for every sequence)."""
        return int(self.T['NPTR'].flatten()[0])

    def _vk(self, S):
        S = S.float().reshape(-1, S.shape[-2], S.shape[-1])
        return (S.transpose(1, 2) if self._key_major_io else S).contiguous()

    @torch.no_grad()
    def load(self, S):
        """Replace the stored state (in place) and empty the buffer."""
        codes, scales = pack_vk(self._vk(S), self.fmt)
        self.T['S'].copy_(codes)
        self.T['SC'].copy_(scales)
        for k in _BUFFER:
            self.T[k].zero_()

    def dequantize(self):
        """The stored state (without the buffered tokens) as fp32."""
        S = unpack_vk(self.T['S'], self.T['SC'], self.fmt, self.DK)
        return S.transpose(1, 2) if self._key_major_io else S

    def stored_bytes(self):
        """Resident bytes by purpose: the state (payload and scales), the decode buffer, the decay bookkeeping."""
        T = self.T
        out = {'state': _nbytes(T['S']) + (_nbytes(T['SC']) if self.fmt is not None else 0),
               'buffer': _nbytes(T['KB']) + _nbytes(T['UB']) + (_nbytes(T['KBS']) + _nbytes(T['UBS']) if self.qbuf else 0),
               'decay': _nbytes(T['GB']) + _nbytes(T['GCUR']) + _nbytes(T['NPTR'])}
        out['total'] = sum(out.values())
        return out
