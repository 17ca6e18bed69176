"""Storage formats of a recurrent state, as far as the packed decode path needs them.

A recurrent state is a float tensor ``[..., d_k, d_v]``.  ``Quantizer`` describes an integer grid with one fp16/fp32
scale per group of consecutive entries along the key axis (``axis='k'``) or the value axis (``axis='v'``); ``fake``
returns the state after a store/load round trip.  Only what a packed store can hold is implemented here: symmetric
round-to-nearest-even without rotation.  The remaining fields exist so that a format object written for the
reference (``statequant.Quantizer``, ``src/statequant/quantizer.py:81-121``) can be passed unchanged and is refused
with the same message when the packed path cannot hold it.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

FP16_TINY = 2.0 ** -24          # smallest fp16 subnormal: floor of a stored scale


class Format:
    def fake(self, S):
        raise NotImplementedError

    def __call__(self, S):
        return self.fake(S)


@dataclass(frozen=True)
class Identity(Format):
    """Full precision (reference: ``quantizer.py:44-53``)."""
    bits: int = 32

    def fake(self, S):
        return S

    def bits_per_value(self, d_k, d_v):
        return float(self.bits)


@dataclass(frozen=True)
class FloatCast(Format):
    """Round trip through a float dtype (reference: ``quantizer.py:56-78``; stochastic rounding is an
    evaluation-only feature and not provided)."""
    dtype: str = 'fp16'
    stochastic: bool = False

    def fake(self, S):
        if self.stochastic:
            raise NotImplementedError('stochastic float casts belong to the fake-quant evaluation path')
        dt = {'bf16': torch.bfloat16, 'fp16': torch.float16, 'fp8': torch.float8_e4m3fn}[self.dtype]
        return S.float().to(dt).to(S.dtype)

    def bits_per_value(self, d_k, d_v):
        return 8.0 if self.dtype == 'fp8' else 16.0


@dataclass(frozen=True)
class Quantizer(Format):
    """Integer state grid with per-group scales (field meaning as the reference's dataclass).

    bits, axis, group   payload width; 'k' = groups of ``group`` consecutive key entries of one value column,
                        'v' = groups of consecutive value entries of one key row; a group that does not divide its
                        axis leaves a shorter last group
    scale_dtype         'fp32': scale used as computed; 'fp16': the scale is rounded to fp16 (and clamped at 2^-24)
                        BEFORE the payload is rounded against it, which is what a packed store holds
    """
    bits: int = 4
    axis: str = 'k'
    group: int = 32
    affine: bool = False
    zero_point: str = 'int'
    rotation: str | None = None
    rounding: str = 'rtn'
    scale_bits: int = 16
    scale_dtype: str = 'fp32'

    def __post_init__(self):
        assert self.axis in ('k', 'v', 'head'), self.axis
        assert 2 <= self.bits <= 15, self.bits
        assert self.scale_bits in (8, 16) and self.scale_dtype in ('fp32', 'fp16')

    @property
    def qmax(self):
        return 2 ** (self.bits - 1) - 1

    def _scale(self, amax):
        s = amax.clamp_min(1e-8) / self.qmax
        if self.scale_dtype == 'fp16':
            s = s.to(torch.float16).float().clamp_min(FP16_TINY)
        return s

    def fake(self, S):
        if self.affine or self.rotation is not None or self.rounding != 'rtn' or self.scale_bits != 16 \
                or self.axis == 'head':
            raise NotImplementedError('only symmetric RTN formats with 16-bit scales are implemented here')
        x = S.float()
        ax = -2 if self.axis == 'k' else -1                       # S is [..., d_k, d_v]
        x = x.movedim(ax, -1)
        n, g = x.shape[-1], self.group
        ng = -(-n // g)
        xp = torch.nn.functional.pad(x, (0, ng * g - n)).reshape(*x.shape[:-1], ng, g)
        s = self._scale(xp.abs().amax(-1, keepdim=True))
        y = (torch.round(xp / s).clamp(-self.qmax, self.qmax) * s).reshape(*x.shape[:-1], ng * g)[..., :n]
        return y.movedim(-1, ax).to(S.dtype)

    def bits_per_value(self, d_k, d_v):
        n = d_k if self.axis == 'k' else d_v
        return self.bits + self.scale_bits * -(-n // self.group) / n
