"""statequant_b200: the fused packed-state decode step of StateQuant as hand-written sm_100a CUDA.

    import statequant_b200 as sq
    lay = sq.kernels.SlotLayout(sq.Quantizer(4, 'k', 64), hv=32, hk=16, dk=128, dv=128, m=8)
    blob = lay.alloc(num_slots); views = lay.views(blob)
    lay.step(views, idx, q, k, v, out, scale, gate=(a, b, A_log, dt_bias))
"""
from .quantizer import FloatCast, Format, Identity, Quantizer
from . import kernels

__version__ = '0.1.0'
__all__ = ['Quantizer', 'FloatCast', 'Identity', 'Format', 'kernels']
