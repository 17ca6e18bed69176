"""Shared machinery of the parity tests: build a slot blob for a case, step it through the oracle (host) or the
CUDA kernels (device), and compare blobs field by field."""
from __future__ import annotations

import os

import numpy as np
import torch

import statequant_b200 as sq
from statequant_b200.kernels import KDASlotLayout, Mamba2SlotLayout, SlotLayout

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')


def layout_of(c):
    fmt = c['fmt'] if isinstance(c['fmt'], str) else sq.Quantizer(*c['fmt'])
    if c['kind'] == 'gdn':
        return SlotLayout(fmt, c['hv'], c['hk'], c['dk'], c['dv'], m=c['m'], buffer_bits=c['bb'])
    if c['kind'] == 'm2':
        return Mamba2SlotLayout(fmt, c['hv'], c['hk'], c['dk'], c['dv'], m=c['m'], buffer_bits=c['bb'])
    return KDASlotLayout(fmt, c['hv'], c['dk'], c['dv'], m=c['m'], buffer_bits=c['bb'])


def fresh_blob(lay, n_slots, seed=0, pad=0):
    """A garbage-filled host blob [n_slots, nbytes + pad] (the kernels must tolerate garbage in dead buffer slots
    and touch nothing outside live slots); returns (raw, blob view)."""
    g = torch.Generator().manual_seed(seed)
    raw = torch.randint(0, 256, (n_slots, lay.nbytes + 2 * pad), dtype=torch.uint8, generator=g)
    return raw, raw[:, pad:pad + lay.nbytes]


def step_args(c, inp, t, dtype=torch.float32):
    """Per-step activations of case c at step t as the layouts' step() takes them."""
    cv = lambda x: x.to(dtype).contiguous()          # noqa: E731
    if c['kind'] == 'gdn':
        return dict(q=cv(inp['q'][t]), k=cv(inp['k'][t]), v=cv(inp['v'][t]), g=inp['g'][t].contiguous(),
                    beta=inp['beta'][t].contiguous())
    if c['kind'] == 'm2':
        return dict(x=cv(inp['x'][t]), dt=cv(inp['dt'][t]), B=cv(inp['Bm'][t]), C=cv(inp['Cm'][t]))
    return dict(q=cv(inp['q'][t]), k=cv(inp['k'][t]), v=cv(inp['v'][t]), g=inp['g'][t].contiguous(),
                beta=inp['beta'][t].contiguous())


def run_step(c, lay, views, idx, a, out, inp, oracle=None):
    """One step through the CUDA kernels (oracle=None) or the oracle module."""
    dev = out.device
    if c['kind'] == 'gdn':
        f = lay.step if oracle is None else (lambda *x, **kw: oracle.gdn_step(lay, *x, **kw))
        return f(views, idx, a['q'], a['k'], a['v'], out, c['dk'] ** -0.5, g=a['g'], beta=a['beta'])
    if c['kind'] == 'm2':
        A, D, dtb = inp['A'].to(dev), inp['D'].to(dev), inp['dt_bias'].to(dev)
        f = lay.step if oracle is None else (lambda *x, **kw: oracle.mamba2_step(lay, *x, **kw))
        sp = c.get('softplus', True)
        return f(views, idx, a['x'], a['dt'], a['B'], a['C'], out, A, D, dtb if sp else None, dt_softplus=sp)
    f = lay.step if oracle is None else (lambda *x, **kw: oracle.kda_step(lay, *x, **kw))
    return f(views, idx, a['q'], a['k'], a['v'], a['g'], a['beta'], out, c['dk'] ** -0.5)


def field_diff(lay, blob_a, blob_b, slots):
    """{field: number of differing elements} between two blobs over the given slots."""
    va, vb = lay.views(blob_a), lay.views(blob_b)
    sl = torch.as_tensor(slots, dtype=torch.long)
    out = {}
    for name in va:
        x, y = va[name][sl], vb[name][sl]
        if x.dtype in (torch.float32, torch.float16, torch.bfloat16):
            x, y = x.view(torch.int32 if x.dtype == torch.float32 else torch.int16), \
                y.view(torch.int32 if y.dtype == torch.float32 else torch.int16)
        out[name] = int((x != y).sum())
    return out


def nibble_steps(a, b):
    """For uint8 tensors of packed 4-bit codes: (number of differing codes, max |difference| in code steps)."""
    al, ah, bl, bh = (a & 15).short(), (a >> 4).short(), (b & 15).short(), (b >> 4).short()
    d = torch.cat([(al - bl).abs().flatten(), (ah - bh).abs().flatten()])
    return int((d != 0).sum()), int(d.max()) if d.numel() else 0


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name + '.npz')))
