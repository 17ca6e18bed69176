"""Slot-addressed packed Gated DeltaNet states and their decode step.

``SlotLayout`` mirrors the reference class of the same name (``src/statequant/kernels/slots.py:40-257``): same
constructor, same ``fields`` / ``nbytes`` / ``views`` / ``alloc`` / ``read`` / ``write`` and the same ``step``
signature, on the same bytes.  ``step`` is one launch of the sm_100a kernel through ``sqb_gdn_step``; ``fused`` is
accepted for compatibility and ignored (there is a single code path).
"""
from __future__ import annotations

import torch

from .. import _cabi
from .formats import pow2
from .layout import KIND_GDN, BlobLayout, set_shape


def _gdn_inputs(idx, q, k, v, out, scale, g, beta, gate, per_key_head):
    """Assemble ``sqb_gdn_inputs_t`` for tensors laid out [rows, heads, dim] (or [rows * heads, dim] for the
    lockstep container, which passes explicit strides through 3-d views)."""
    a = _cabi.GdnInputs()
    rows = out.shape[0]
    a.idx = _cabi.ptr(idx)
    a.q, a.sq = q.data_ptr(), _cabi.row_stride_bytes(q)
    a.k, a.sk = k.data_ptr(), _cabi.row_stride_bytes(k)
    a.v, a.sv = v.data_ptr(), _cabi.row_stride_bytes(v)
    a.qk_dtype, a.v_dtype = _cabi.dtype_code(q), _cabi.dtype_code(v)
    assert k.dtype == q.dtype
    if gate is not None:
        ga, gb, A_log, dt_bias = gate
        assert ga.stride(-1) == 1 and gb.stride(-1) == 1 and ga.dtype == gb.dtype
        assert A_log.is_contiguous() and dt_bias.is_contiguous()
        a.a, a.sa, a.b, a.sb = ga.data_ptr(), _cabi.row_stride_bytes(ga), gb.data_ptr(), _cabi.row_stride_bytes(gb)
        a.A_log, a.dt_bias = A_log.data_ptr(), dt_bias.data_ptr()
        a.ab_dtype, a.alog_dtype, a.dtb_dtype = _cabi.dtype_code(ga), _cabi.dtype_code(A_log), _cabi.dtype_code(dt_bias)
        a.gate = 1
    else:
        assert g.stride(-1) == 1 and beta.stride(-1) == 1 and g.dtype == beta.dtype
        a.g, a.sg, a.beta, a.sbeta = g.data_ptr(), _cabi.row_stride_bytes(g), beta.data_ptr(), _cabi.row_stride_bytes(beta)
        a.gb_dtype = _cabi.dtype_code(g)
        a.gate = 0
    a.out, a.so, a.out_dtype = out.data_ptr(), _cabi.row_stride_bytes(out), _cabi.dtype_code(out)
    a.scale, a.rows, a.qk_per_key_head = float(scale), rows, int(per_key_head)
    return a


class SlotLayout(BlobLayout):
    """The packed per-slot layout of one GDN layer and the operations on a batch of slots.

    fmt          ``Quantizer(4 or 8, 'k' or 'v', group)``, 'bf16' or 'fp32' (an unpacked float state)
    hv, hk       value / key heads of the layer (on this rank); hv % hk == 0
    dk, dv       head dims
    m            buffer length (power of two): the state is folded and re-rounded every m tokens
    buffer_bits  8 (int8 + fp16 scale per vector) or 16 (bf16)
    fused        ignored (kept so that reference call sites need no change)
    """
    kind = KIND_GDN

    def __init__(self, fmt, hv, hk, dk, dv, m=8, buffer_bits=8, fused=None):
        self.fused = fused
        full = fmt == 'fp32' if isinstance(fmt, str) else False
        self.state_dtype = torch.float32 if full else torch.bfloat16
        set_shape(self, 'bf16' if full else fmt, hv, hk, dk, dv, m, buffer_bits, gdn_dims=True, float_group=32)
        self.DKP, self.DVP = pow2(dk), pow2(dv)
        self._finish()

    def step(self, views, idx, q, k, v, out, scale, *, g=None, beta=None, gate=None, fused='layout'):
        """One decode token for every batch row b, on slot ``idx[b]`` (int32 [B]; <= 0 = padding row: the output
        row is zeroed and nothing else is touched).

        q, k    [B, hk, d_k] per key head, raw (l2-normalised in the kernel); any row stride, unit inner stride
        v       [B, hv, d_v];  out [B, hv, d_v] contiguous, written
        g, beta [B, hv] log decay and beta after the sigmoid; or ``gate=(a, b, A_log, dt_bias)`` to form
                g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b) in the kernel
        One kernel launch on the current stream; no allocation, no host sync (CUDA-graph capturable).
        """
        B = idx.shape[0]
        if B == 0:
            return out
        assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
        assert q.stride(-2) == self.DK and k.stride(-2) == self.DK and v.stride(-2) == self.DV
        assert out.is_contiguous() and out.shape[0] >= B
        assert idx.dtype == torch.int32 and idx.is_contiguous()
        a = _gdn_inputs(idx, q, k, v, out[:B], scale, g, beta, gate, True)
        st = self._struct(views)
        _cabi.check(_cabi.lib().sqb_gdn_step(_cabi.C.byref(st), _cabi.C.byref(a), _cabi.current_stream(q.device)),
                    'sqb_gdn_step')
        return out
