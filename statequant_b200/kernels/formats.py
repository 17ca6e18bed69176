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


def packed_format(fmt):
    """The format a packed store holds for ``fmt``: the same quantizer with fp16 scales, or ``None`` for a bf16
    state ('bf16', ``FloatCast('bf16')`` or None).  Anything a packed store cannot hold is refused
    (reference: ``fold.py:91-104``).  ``fmt`` may be this package's ``Quantizer`` or any dataclass with the same
    fields (the reference's own)."""
    if fmt is None or (isinstance(fmt, str) and fmt == 'bf16'):
        return None
    if getattr(fmt, 'dtype', None) == 'bf16' and hasattr(fmt, 'stochastic') and not fmt.stochastic:
        return None
    need = ('bits', 'axis', 'group', 'affine', 'rotation', 'rounding', 'scale_bits')
    assert all(hasattr(fmt, a) for a in need), f'packed storage needs a Quantizer or bf16, got {fmt!r}'
    assert fmt.bits in (4, 8) and fmt.axis in ('k', 'v'), (fmt.bits, fmt.axis)
    assert not fmt.affine and fmt.rotation is None and fmt.rounding == 'rtn' and fmt.scale_bits == 16, \
        'packed storage implements symmetric RTN with 16-bit scales and no rotation'
    assert fmt.group % 2 == 0
    return dataclasses.replace(fmt, scale_dtype='fp16')


def state_bits(fmt):
    return 16 if fmt is None else fmt.bits


def pow2(n):
    """Smallest power of two >= n."""
    return 1 << max(0, (int(n) - 1).bit_length())


def check_dims(fmt, dk, dv):
    """Head dims and groups a packed GDN store accepts (reference: ``fold.py:63-76``)."""
    assert dk >= 16 and dk % 2 == 0, f'd_k must be even and >= 16, got {dk}'
    assert dv % 32 == 0, f'd_v must be a multiple of 32, got {dv}'
    if fmt is not None:
        g = fmt.group
        assert g >= 2 and g & (g - 1) == 0, f'group {g} must be a power of two'
        if fmt.axis == 'k':
            assert g <= pow2(dk) and pow2(dk) // g <= 8, f'key group {g} on d_k {dk}: 1 .. 8 groups'
        else:
            assert dv % g == 0, f'value group {g} must divide d_v {dv}'


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
