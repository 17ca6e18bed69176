"""Byte layout of one layer's per-slot state blob, shared by the GDN, Mamba2 and KDA layouts.

A serving engine keeps every running sequence's recurrent state in one slot of a preallocated cache and hands each
step a table of slot indices.  A slot is a byte blob; its fields, in this order and each padded to 16 bytes, are
(reference: ``src/statequant/kernels/slots.py:9-28,76-95``, ``mamba2.py:359-370``, ``kda.py:311-323``)

    GB    fp32  [HV, m] (KDA: [HV, m, d_k])   cumulative log decay of each buffered token
    GCUR  fp32  [HV]    (KDA: [HV, d_k])      running log decay since the last fold
    NPTR  int32 [max(HV, 4)]                  buffer fill counter, one copy per value head
    SC    fp16  scales (integer states only)  axis 'k': [HV, d_v, ceil(d_k/g)]; axis 'v': [HV, d_v/g, d_k]
    KBS   fp16  [HK, m], UBS fp16 [HV, m]     buffer scales (int8 buffer only)
    S     codes uint8 [HV, d_v, d_k/2] | int8 [HV, d_v, d_k] | bf16 / fp32 [HV, d_v, d_k]
    KB    int8 / bf16 [HK, m, d_k]            buffered keys, per KEY head (Mamba2: per group)
    UB    int8 / bf16 [HV, m, d_v]            buffered delta values

so a blob written by the reference can be stepped by these kernels and the other way round.
"""
from __future__ import annotations

import ctypes
import math

import torch

from .. import _cabi
from .formats import pack_vk, unpack_vk

ALIGN = 16
KIND_GDN, KIND_M2, KIND_KDA = 0, 1, 2


def _esize(dt):
    return torch.empty((), dtype=dt).element_size()


def field_table(specs):
    """[(name, dtype, shape)] -> ({name: (offset, dtype, shape, nbytes)}, total bytes), 16-byte aligned fields."""
    table, off = {}, 0
    for name, dt, shape in specs:
        nb = math.prod(shape) * _esize(dt)
        table[name] = (off, dt, tuple(shape), nb)
        off += -(-nb // ALIGN) * ALIGN
    return table, off


def state_specs(fmt, state_dtype, hv, hk, dk, dv, m, qbuf, decay_width=1, ragged=True):
    """The field list of one slot.  ``decay_width`` is d_k for KDA (per-channel decays), else 1."""
    bdt = torch.int8 if qbuf else torch.bfloat16
    gshape = (hv, m) if decay_width == 1 else (hv, m, decay_width)
    cshape = (hv,) if decay_width == 1 else (hv, decay_width)
    specs = [('GB', torch.float32, gshape), ('GCUR', torch.float32, cshape), ('NPTR', torch.int32, (max(hv, 4),))]
    if fmt is None:
        sdt, sshape = state_dtype, (hv, dv, dk)
    else:
        g = fmt.group
        ng = -(-dk // g) if ragged else dk // g
        specs.append(('SC', torch.float16, (hv, dv, ng) if fmt.axis == 'k' else (hv, dv // g, dk)))
        sdt = torch.uint8 if fmt.bits == 4 else torch.int8
        sshape = (hv, dv, dk // 2) if fmt.bits == 4 else (hv, dv, dk)
    if qbuf:
        specs += [('KBS', torch.float16, (hk, m)), ('UBS', torch.float16, (hv, m))]
    specs += [('S', sdt, sshape), ('KB', bdt, (hk, m, dk)), ('UB', bdt, (hv, m, dv))]
    return specs


def state_struct(tables, strides, *, bits, axis_k, group, buffer_bits, m, hv, hk, dk, dv):
    """Fill a ``sqb_state_t`` from per-sequence tensors ``tables[name]`` and byte strides ``strides[name]``."""
    st = _cabi.State()
    for name, fld, sfld in (('S', 'S', 'sS'), ('SC', 'SC', 'sSC'), ('KB', 'KB', 'sKB'), ('KBS', 'KBS', 'sKBS'),
                            ('UB', 'UB', 'sUB'), ('UBS', 'UBS', 'sUBS'), ('GB', 'GB', 'sGB'),
                            ('GCUR', 'GCUR', 'sGC'), ('NPTR', 'NPTR', 'sN')):
        t = tables.get(name)
        setattr(st, fld, None if t is None else t.data_ptr())
        setattr(st, sfld, 0 if t is None else int(strides[name]))
    st.bits, st.axis_k, st.group, st.buffer_bits, st.m = bits, int(axis_k), group, buffer_bits, m
    st.hv, st.hk, st.dk, st.dv = hv, hk, dk, dv
    return st


def set_shape(obj, fmt, hv, hk, dk, dv, m, buffer_bits, *, gdn_dims, float_group):
    """Store on ``obj`` the attributes every layout and container carries (fmt, bits, HV, HK, DK, DV, m, gqa,
    buffer_bits, qbuf, axk, group) after checking that the kernels have a tiling for them.

    gdn_dims     True: the Gated DeltaNet rules of ``check_dims`` (padded key rows, at most 8 groups per row, any m);
                 False: the Mamba2 / KDA rules (the groups tile the quantised axis exactly, m <= 32)
    float_group  the group written into the state struct when the state is a float one (never read by a kernel)"""
    from .formats import _need, check_dims, packed_format, pow2, state_bits
    obj.fmt = packed_format(fmt)
    obj.bits = state_bits(obj.fmt)
    _need(hk >= 1 and hv % hk == 0, f'{hv} value heads do not divide over {hk} key heads')
    _need(m >= 1 and m == pow2(m) and (gdn_dims or m <= 32),
          f'm = {m}: the buffer length is a power of two' + ('' if gdn_dims else ' of at most 32'))
    _need(buffer_bits in (8, 16), f'buffer_bits = {buffer_bits}: the decode buffer is int8 or bf16')
    if gdn_dims:
        check_dims(obj.fmt, dk, dv)
    else:
        _need(dk % 2 == 0 and dk >= 16, f'd_k = {dk}: need an even width of at least 16')
        if obj.fmt is not None:
            g, along = obj.fmt.group, dk if obj.fmt.axis == 'k' else dv
            _need(g >= 2 and g == pow2(g), f'group = {g}: need a power of two')
            _need(along % g == 0, f'group = {g} does not tile d_{obj.fmt.axis} = {along}')
    obj.HV, obj.HK, obj.DK, obj.DV, obj.m, obj.gqa = hv, hk, dk, dv, m, hv // hk
    obj.buffer_bits, obj.qbuf = buffer_bits, buffer_bits == 8
    obj.axk = obj.fmt is not None and obj.fmt.axis == 'k'
    obj.group = obj.fmt.group if obj.fmt is not None else float_group


def describe_format(obj):
    """'int4 x k/32' style tag of a layout's state format."""
    if obj.fmt is None:
        return 'fp32' if getattr(obj, 'state_dtype', None) == torch.float32 else 'bf16'
    return f'int{obj.bits} x {obj.fmt.axis}/{obj.group}'


class BlobLayout:
    """Common part of the slot layouts: field table, typed views, allocation, the ``sqb_state_t`` of a blob and
    the torch read / write used around prefill."""

    kind = KIND_GDN
    _head_words = ('hv', 'hk', 'dk', 'dv')          # how the subclass names HV, HK, DK, DV in its constructor

    def __repr__(self):
        dims = ', '.join(f'{w}={x}' for w, x in zip(self._head_words, (self.HV, self.HK, self.DK, self.DV)) if w)
        buf = 'int8' if self.qbuf else 'bf16'
        return f'<{type(self).__name__} {describe_format(self)} | {dims} | {self.m} x {buf} buffer | {self.nbytes} B per slot>'

    def _finish(self, decay_width=1, ragged=True):
        self.fields, self.nbytes = field_table(state_specs(
            self.fmt, self.state_dtype, self.HV, self.HK, self.DK, self.DV, self.m, self.qbuf, decay_width, ragged))
        self._structs = {}

    # -- bytes --------------------------------------------------------------------------------------------
    def breakdown(self):
        """Bytes per slot by field, before alignment padding."""
        return {n: f[3] for n, f in self.fields.items()}

    def views(self, blob):
        """uint8 ``[num_slots, >= nbytes]`` with unit inner stride, a slot stride and a base address that are
        multiples of 16 -> {field: typed view [num_slots, *shape]} (reference: ``slots.py:108-117``)."""
        assert blob.dtype == torch.uint8 and blob.dim() == 2 and blob.shape[1] >= self.nbytes, blob.shape
        assert blob.stride(1) == 1 and blob.stride(0) % ALIGN == 0 and blob.data_ptr() % ALIGN == 0
        n = blob.shape[0]
        return {name: blob[:, off:off + nb].view(dt).view(n, *shape)
                for name, (off, dt, shape, nb) in self.fields.items()}

    def alloc(self, num_slots, device='cuda'):
        """A zeroed standalone blob ``[num_slots, nbytes]``."""
        return torch.zeros(num_slots, self.nbytes, dtype=torch.uint8, device=device)

    def _struct(self, views):
        """The ``sqb_state_t`` of a views dict (cached on the blob's address and slot stride)."""
        S = views['S']
        key = (S.data_ptr(), S.stride(0), S.shape[0])
        st = self._structs.get(key)
        if st is None:
            strides = {n: v.stride(0) * v.element_size() for n, v in views.items()}
            st = state_struct(views, strides, bits=self.bits if self.fmt is not None else
                              (32 if self.state_dtype == torch.float32 else 16),
                              axis_k=self.axk, group=self.group, buffer_bits=self.buffer_bits, m=self.m,
                              hv=self.HV, hk=self.HK, dk=self.DK, dv=self.DV)
            if len(self._structs) > 64:
                self._structs.clear()
            self._structs[key] = st
        return st

    # -- prefill side: device kernels for CUDA blobs of the 4 / 8-bit formats, torch otherwise -------------------
    def _device_io(self, views):
        """True if the slot read / write kernels take this layout and blob (4 / 8-bit state, d_k 64 or 128, groups
        the kernels support, blob on a GPU)."""
        if self.fmt is None or not views['S'].is_cuda or self.DK not in (64, 128):
            return False
        g = self.group
        if self.axk:
            return g % 16 == 0 and self.DK % g == 0
        rpp = 32 // (self.DK // 16)
        return g % rpp == 0 and self.DV % g == 0 and self.DV % (4 * rpp) == 0 and g // (rpp * min(4, g // rpp)) <= 2

    @torch.no_grad()
    def read(self, views, idx):
        """Current state of slots ``idx`` as fp32 ``[P, HV, d_v, d_k]``: the stored state advanced across its
        pending buffer, S_n = a_n S_0 + sum_{i<n} (a_n / a_i) u_i k_i^T (KDA: the decays per key channel).
        Slots holding garbage give garbage.  Reference: ``slots.py:210-233``, ``kda.py:351-372``."""
        if self._device_io(views):
            i32 = idx.to(torch.int32).contiguous()
            out = torch.empty(i32.shape[0], self.HV, self.DV, self.DK, dtype=torch.float32, device=i32.device)
            _cabi.check(_cabi.lib().sqb_slot_read(ctypes.byref(self._struct(views)), self.kind, i32.data_ptr(),
                                                  i32.shape[0], out.data_ptr(), _cabi.current_stream(i32.device)), 'sqb_slot_read')
            return out
        idx = idx.long()
        P, m = idx.shape[0], self.m
        V = views
        codes = V['S'][idx].flatten(0, 1)
        sc = V['SC'][idx].flatten(0, 1) if 'SC' in V else None
        S0 = unpack_vk(codes, sc, self.fmt, self.DK).view(P, self.HV, self.DV, self.DK)
        kb, ub = V['KB'][idx].float(), V['UB'][idx].float()                        # [P, HK, m, DK], [P, HV, m, DV]
        if self.qbuf:
            kb = kb * V['KBS'][idx].float()[..., None]
            ub = ub * V['UBS'][idx].float()[..., None]
        n = V['NPTR'][idx, 0] & (m - 1)
        live = torch.arange(m, device=idx.device)[None, :] < n[:, None]            # [P, m]
        gcur, gb = V['GCUR'][idx], V['GB'][idx]
        kb = kb.repeat_interleave(self.HV // self.HK, dim=1)                       # [P, HV, m, DK]
        if self.kind == KIND_KDA:
            lv = live[:, None, :, None]
            dec = torch.where(lv, torch.exp(gcur[:, :, None, :] - torch.where(lv, gb, 0.)), 0.)
            kd = torch.where(lv, kb, 0.) * dec
            return torch.exp(gcur)[:, :, None, :] * S0 + torch.einsum('phmv,phmk->phvk', torch.where(lv, ub, 0.), kd)
        lv = live[:, None, :]
        dec = torch.where(lv, torch.exp(gcur[..., None] - torch.where(lv, gb, 0.)), 0.)
        ub = torch.where(lv[..., None], ub, 0.) * dec[..., None]
        kb = torch.where(lv[..., None], kb, 0.)
        return torch.exp(gcur)[..., None, None] * S0 + torch.einsum('phmv,phmk->phvk', ub, kb)

    @torch.no_grad()
    def write(self, views, idx, S):
        """Store states ``S [P, HV, d_v, d_k]`` packed into slots ``idx`` and empty their buffers (counter and
        running decay zeroed).  Reference: ``slots.py:236-252``."""
        if self._device_io(views):
            i32 = idx.to(torch.int32).contiguous()
            X = S.reshape(i32.shape[0], self.HV, self.DV, self.DK).to(device=i32.device, dtype=torch.float32).contiguous()
            _cabi.check(_cabi.lib().sqb_slot_write(ctypes.byref(self._struct(views)), self.kind, i32.data_ptr(),
                                                   i32.shape[0], X.data_ptr(), _cabi.current_stream(i32.device)), 'sqb_slot_write')
            return
        idx = idx.long()
        P = idx.shape[0]
        V = views
        if self.fmt is None and self.state_dtype == torch.float32:
            V['S'][idx] = S.reshape(P, *V['S'].shape[1:]).float()
        else:
            codes, sc = pack_vk(S.reshape(P * self.HV, self.DV, self.DK), self.fmt)
            V['S'][idx] = codes.view(P, *V['S'].shape[1:])
            if 'SC' in V:
                V['SC'][idx] = sc.view(P, *V['SC'].shape[1:])
        V['NPTR'][idx] = 0
        V['GCUR'][idx] = 0.

    def stored(self, views, idx):
        """(codes, scales) of slots ``idx``."""
        idx = idx.long()
        return views['S'][idx], (views['SC'][idx] if 'SC' in views else None)
