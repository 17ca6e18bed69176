"""The short causal convolution in front of the decode step (one token per sequence), on the sm_100a kernel.

``causal_conv1d_update`` takes the arguments of the op the reference's vLLM forward calls right before ``lay.step``
(``src/statequant/integrations/vllm_plugin.py:379-381``; vLLM's ``model_executor/layers/mamba/ops/causal_conv1d.py``)
for the plain decode case: one token per row, no speculative decoding, no prefix-cache block indices.  Its output rows
are ``q | k | v``; ``split_qkv`` gives the column slices the step reads in place.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _cabi

NULL_BLOCK_ID = 0      # vLLM's null block: rows that point at it are padding


def causal_conv1d_update(x, conv_state, weight, bias=None, activation=None, conv_state_indices=None,
                         num_accepted_tokens=None, query_start_loc=None, max_query_len=-1,
                         null_block_id=NULL_BLOCK_ID, block_idx_last_scheduled_token=None, initial_state_idx=None,
                         validate_data=False):
    """x [rows, dim] (or [rows, dim, 1]) -> the convolved row, in place (the same tensor is returned).

    conv_state [lines, dim, state_len] with any strides (vLLM passes the transposed view of a [lines, state_len, dim]
    cache), state_len >= width - 1; weight [dim, width]; bias [dim] or None; activation None / 'silu' / 'swish' /
    bool; conv_state_indices int32 [rows] or None (row r uses line r).  A row whose line is ``null_block_id`` (or
    negative) is left untouched, and so is its cache line.  x is cast to the state's dtype if it differs (then the
    result is a new tensor in x's dtype, as in vLLM's wrapper)."""
    assert num_accepted_tokens is None and query_start_loc is None and block_idx_last_scheduled_token is None and \
        initial_state_idx is None, 'causal_conv1d_update: the plain one-token decode case only'
    if isinstance(activation, bool):
        activation = 'silu' if activation else None
    assert activation in (None, 'silu', 'swish'), f'activation {activation!r}'
    assert x.is_cuda and conv_state.is_cuda and weight.is_cuda, 'causal_conv1d_update runs on CUDA tensors'
    x0 = x
    squeeze = x.dim() == 3
    if squeeze:
        assert x.size(-1) == 1, 'one token per row'
        x = x.squeeze(-1)
    if x.dtype != conv_state.dtype:
        x = x.to(conv_state.dtype)
    assert x.dim() == 2 and x.stride(1) == 1, 'x: [rows, dim] with unit inner stride'
    rows, dim = x.shape
    width = weight.size(1)
    lines, sdim, state_len = conv_state.shape
    assert weight.size(0) == dim and sdim == dim, 'dim of x, weight and conv_state differ'
    if bias is not None:
        assert bias.dtype == weight.dtype and bias.is_contiguous() and bias.numel() == dim
    idx = conv_state_indices
    if idx is not None:
        assert idx.numel() == rows
        if idx.dtype != torch.int32 or not idx.is_contiguous():
            idx = idx.to(torch.int32).contiguous()
    else:
        assert lines >= rows
    es, ws = x.element_size(), weight.element_size()
    a = _cabi.ConvUpdate(
        x=x.data_ptr(), sx=x.stride(0) * es, out=x.data_ptr(), so=x.stride(0) * es,
        state=conv_state.data_ptr(), s_line=conv_state.stride(0) * es, s_dim=conv_state.stride(1) * es,
        s_tok=conv_state.stride(2) * es, w=weight.data_ptr(), sw_dim=weight.stride(0) * ws,
        sw_tap=weight.stride(1) * ws, bias=_cabi.ptr(bias), idx=_cabi.ptr(idx), rows=rows, dim=dim, width=width,
        state_len=state_len, x_dtype=_cabi.dtype_code(x), w_dtype=_cabi.dtype_code(weight),
        silu=int(activation is not None), null_line=-1 if null_block_id is None else int(null_block_id))
    _cabi.check(_cabi.lib().sqb_conv1d_update(C.byref(a), _cabi.current_stream(x.device)), 'sqb_conv1d_update')
    if x.data_ptr() != x0.data_ptr():
        x = x.to(x0.dtype)
    return x.unsqueeze(-1) if squeeze else x


def split_qkv(x, hk, dk, hv, dv):
    """The convolved rows [rows, 2 hk dk + hv dv] as the step's q [rows, hk, dk], k, v [rows, hv, dv]: views, no copy."""
    kd = hk * dk
    return (x[:, :kd].unflatten(1, (hk, dk)), x[:, kd:2 * kd].unflatten(1, (hk, dk)),
            x[:, 2 * kd:].unflatten(1, (hv, dv)))
