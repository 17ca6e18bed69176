"""Packed storage formats: which formats a packed state can hold, and the torch-side pack / unpack.

``pack_vk`` / ``unpack_vk`` are the definition of the stored bytes: ``unpack(pack(S, q))`` equals
``Quantizer(..., scale_dtype='fp16').fake(S)`` element for element (reference: ``src/statequant/kernels/fold.py:91-173``).
They run in torch on any device and are used on the prefill side (``write``) and by tests; the decode step itself
never goes through them.

Stored orientation is value-major, ``[heads, d_v, d_k]`` with d_k contiguous.  Four-bit codes pack two per byte
along d_k: byte j holds ``code[2j] + 8`` in its low nibble and ``code[2j+1] + 8`` in its high nibble.  Scales are
fp16: axis 'k' ``[heads, d_v, ceil(d_k/group)]``, axis 'v' ``[heads, d_v/group, d_k]``.
"""
from __future__ import annotations

import dataclasses

import torch

from ..quantizer import FP16_TINY, FloatCast, Quantizer


_QUANTIZER_FIELDS = ('bits', 'axis', 'group', 'affine', 'rotation', 'rounding', 'scale_bits')


def _need(ok, why):
    if not ok:
        raise AssertionError(why)


def packed_format(fmt):
    """What a packed store keeps for ``fmt``.  'bf16', ``FloatCast('bf16')`` (not stochastic) and None mean a bf16
    state and give None; a quantizer gives the same quantizer with fp16 scales.  The kernels implement symmetric
    round-to-nearest int4 / int8 with one 16-bit scale per group along d_k or d_v and nothing else, so every other
    quantizer is refused here rather than stored wrongly (reference: ``fold.py:91-104``).  ``fmt`` may be this
    package's ``Quantizer`` or any dataclass with the same fields (the reference's own)."""
    if fmt is None or fmt == 'bf16':
        return None
    if getattr(fmt, 'dtype', None) == 'bf16' and getattr(fmt, 'stochastic', True) is False:
        return None
    missing = [f for f in _QUANTIZER_FIELDS if not hasattr(fmt, f)]
    _need(not missing, f'a packed store holds a Quantizer or bf16; {fmt!r} lacks {missing}')
    _need(fmt.bits in (4, 8), f'state codes are 4 or 8 bits wide, not {fmt.bits}')
    _need(fmt.axis in ('k', 'v'), f"scale groups run along 'k' or 'v', not {fmt.axis!r}")
    _need(fmt.group % 2 == 0, f'group {fmt.group}: two int4 codes share a byte, so groups are even')
    for field, want in (('affine', False), ('rotation', None), ('rounding', 'rtn'), ('scale_bits', 16)):
        _need(getattr(fmt, field) == want, f'{field}={getattr(fmt, field)!r} is not stored packed (only {want!r})')
    return dataclasses.replace(fmt, scale_dtype='fp16')


def state_bits(fmt):
    return 16 if fmt is None else fmt.bits


def pow2(n):
    """Smallest power of two >= n."""
    return 1 << max(0, (int(n) - 1).bit_length())


def check_dims(fmt, dk, dv):
    """Refuse head dims and groups the kernels have no tiling for (reference: ``fold.py:63-76``): a key row is
    padded to a power of two and cut into at most 8 scale groups; the value rows are dealt out 32 at a time."""
    _need(dk % 2 == 0 and dk >= 16, f'd_k = {dk}: need an even width of at least 16')
    _need(dv % 32 == 0, f'd_v = {dv}: need a multiple of 32')
    if fmt is None:
        return
    g, width = fmt.group, pow2(dk)
    _need(g >= 2 and g == pow2(g), f'group = {g}: need a power of two')
    if fmt.axis == 'k':
        _need(g <= width and width <= 8 * g, f'group = {g} along d_k = {dk}: need between 1 and 8 groups per row')
    else:
        _need(dv % g == 0, f'group = {g} along d_v = {dv}: the groups must tile the rows exactly')


def _scale_of(amax, qmax):
    # tensor / tensor: an IEEE division on every device (torch's CUDA kernels turn tensor / python-scalar into a
    # multiplication by the reciprocal, which moves about one scale in a thousand by an fp16 ulp)
    q = torch.full((), qmax, dtype=torch.float32, device=amax.device)
    s = torch.div(amax.clamp_min(1e-8), q).to(torch.float16).float()
    return s.clamp_min(FP16_TINY)


def pack_vk(x, fmt):
    """Value-major float states ``[..., d_v, d_k]`` -> (codes, scales) as stored (see the module docstring).
    A bf16 format returns (bf16 values, a one-element fp16 tensor of ones)."""
    fmt = packed_format(fmt)
    x = x.float().reshape(-1, x.shape[-2], x.shape[-1])
    n, dv, dk = x.shape
    if fmt is None:
        return x.to(torch.bfloat16).contiguous(), torch.ones(1, device=x.device, dtype=torch.float16)
    g, qmax = fmt.group, float(2 ** (fmt.bits - 1) - 1)
    if fmt.axis == 'k':
        ng = -(-dk // g)
        xg = torch.nn.functional.pad(x, (0, ng * g - dk)).view(n, dv, ng, g)       # zero padding: same absmax
        s = _scale_of(xg.abs().amax(3, keepdim=True), qmax)
        c = torch.round(xg / s).clamp_(-qmax, qmax).view(n, dv, ng * g)[..., :dk]
        scales = s.view(n, dv, ng)
    else:
        assert dv % g == 0, f'value group {g} must divide d_v {dv}'
        xg = x.view(n, dv // g, g, dk)
        s = _scale_of(xg.abs().amax(2, keepdim=True), qmax)
        c = torch.round(xg / s).clamp_(-qmax, qmax).view(n, dv, dk)
        scales = s.view(n, dv // g, dk)
    c = c.to(torch.int8)
    if fmt.bits == 4:
        u = (c + 8).to(torch.uint8)
        c = u[..., 0::2] | (u[..., 1::2] << 4)
    return c.contiguous(), scales.to(torch.float16).contiguous()


def unpack_vk(codes, scales, fmt, d_k):
    """Inverse of ``pack_vk``: fp32 ``[n, d_v, d_k]``."""
    fmt = packed_format(fmt)
    if fmt is None:
        return codes.float()
    n, dv = codes.shape[:2]
    if fmt.bits == 4:
        b = codes.to(torch.int16)
        x = torch.stack(((b & 15) - 8, (b >> 4) - 8), -1).view(n, dv, d_k).float()
    else:
        x = codes.float()
    s = scales.float()
    if fmt.axis == 'k':
        return x * s.repeat_interleave(fmt.group, -1)[..., :d_k]
    g = fmt.group
    return (x.view(n, dv // g, g, d_k) * s[:, :, None, :]).view(n, dv, d_k)


def pack(S, fmt):
    """Key-major states ``[..., d_k, d_v]`` (the HF / fla orientation) -> (codes, scales)."""
    return pack_vk(S.float().reshape(-1, S.shape[-2], S.shape[-1]).transpose(1, 2), fmt)


def unpack(codes, scales, fmt, d_k):
    """Inverse of ``pack``: fp32 ``[n, d_k, d_v]``."""
    return unpack_vk(codes, scales, fmt, d_k).transpose(1, 2).contiguous()


def l2norm(x):
    """fla's normalisation, epsilon inside the square root (reference: ``fold.py:181-183``)."""
    x = x.float()
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
