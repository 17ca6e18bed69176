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


_DEVCONST = {}


def run_step(c, lay, views, idx, a, out, inp, oracle=None):
    """One step through the CUDA kernels (oracle=None) or the oracle module."""
    dev = out.device
    if c['kind'] == 'gdn':
        f = lay.step if oracle is None else (lambda *x, **kw: oracle.gdn_step(lay, *x, **kw))
        return f(views, idx, a['q'], a['k'], a['v'], out, c['dk'] ** -0.5, g=a['g'], beta=a['beta'])
    if c['kind'] == 'm2':
        key = (id(inp['A']), str(dev))
        if key not in _DEVCONST:                       # per-layer constants live on the device once (graph capture)
            _DEVCONST[key] = (inp['A'].to(dev), inp['D'].to(dev), inp['dt_bias'].to(dev), inp['A'])
        A, D, dtb = _DEVCONST[key][:3]
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


def _tt(a, dev):
    t = torch.from_numpy(a)
    return t.to(dev)


def replay_vs_golden(name, c, oracle=None, device='cpu', act_dtype=torch.float32):
    """Step a blob through the oracle (``oracle`` given) or the CUDA kernels (``oracle=None``) and compare every
    step with the reference's golden record, adopting the golden buffer entry / folded codes after each comparison
    (so a rounding flip is counted once).  Returns the statistics dict; structural properties are asserted here."""
    from cases import make_inputs
    G = load_golden(name)
    inp = make_inputs(c)
    lay = layout_of(c)
    B, hv, hk, dk, dv, m, T = c['B'], c['hv'], c['hk'], c['dk'], c['dv'], c['m'], c['T']
    raw, blob = fresh_blob(lay, B + 2, seed=c['seed'], pad=64)
    raw = raw.to(device)
    blob = raw[:, 64:64 + lay.nbytes]
    V = lay.views(blob)
    sl = torch.arange(1, B + 1, device=device)
    lay.write(V, sl, inp['S0'].view(B, hv, dv, dk).to(device))
    codes0 = torch.from_numpy(G['codes0'])
    if codes0.dtype == torch.int16:
        codes0 = codes0.view(torch.bfloat16)
    assert torch.equal(V['S'][sl].reshape(codes0.shape).cpu(), codes0)
    idx = torch.arange(1, B + 1, dtype=torch.int32, device=device)
    before = raw.clone()
    st = dict(worst=0., flips=0, nbuf=0, cflips=0, ncodes=0, sflips=0)
    folds = list(G['fold_t'])
    soft = c['kind'] == 'm2' and c.get('softplus', True)
    for t in range(T):
        n = int(V['NPTR'][1, 0])
        out = torch.full((B, hv, dv), 7., device=device)
        a = {k: v.to(device) for k, v in step_args(c, inp, t, act_dtype).items()}
        run_step(c, lay, V, idx, a, out, inp, oracle=oracle)
        want = _tt(G['o'][t], device).view(B, hv, dv)
        st['worst'] = max(st['worst'], ((out - want).abs().max() / want.abs().max()).item())
        kc, uc = _tt(G['Kc'][t], device), _tt(G['Uc'][t], device)
        if c['bb'] == 16:
            kc, uc = kc.view(torch.bfloat16), uc.view(torch.bfloat16)
        st['flips'] += int((V['KB'][sl, :, n].reshape(kc.shape) != kc).sum()) + \
            int((V['UB'][sl, :, n].reshape(uc.shape) != uc).sum())
        st['nbuf'] += kc.numel() + uc.numel()
        if c['bb'] == 8:
            st['sflips'] += int((V['KBS'][sl, :, n].reshape(-1) != _tt(G['Ks'][t], device).reshape(-1)).sum())
            st['sflips'] += int((V['UBS'][sl, :, n].reshape(-1) != _tt(G['Us'][t], device).reshape(-1)).sum())
        gb, gw = V['GB'][sl, :, n].reshape(-1), _tt(G['G'][t], device).reshape(-1)
        if soft or oracle is None:
            # a decay that comes out of exp / log (in-kernel softplus) or is read back from the device differs from
            # torch's in the last place at most; the additions themselves are the same
            assert torch.allclose(gb, gw, rtol=2e-6, atol=1e-12), (gb - gw).abs().max()
        if not soft:
            assert torch.equal(gb, gw)
        V['GB'][sl, :, n] = gw.view(V['GB'][sl, :, n].shape)
        if soft and t not in folds:
            V['GCUR'][sl] = gw.view(V['GCUR'][sl].shape)
        V['KB'][sl, :, n] = kc.view(B, hk, dk)
        V['UB'][sl, :, n] = uc.view(B, hv, dv)
        if c['bb'] == 8:
            V['KBS'][sl, :, n] = _tt(G['Ks'][t], device).view(B, hk)
            V['UBS'][sl, :, n] = _tt(G['Us'][t], device).view(B, hv)
        if t in folds:
            fi = folds.index(t)
            assert int(V['NPTR'][1, 0]) == 0 and float(V['GCUR'][sl].abs().max()) == 0.
            gc = torch.from_numpy(G['codes'][fi])
            if gc.dtype == torch.int16:
                gc = gc.view(torch.bfloat16)
            gc = gc.to(device)
            st['cflips'] += int((V['S'][sl].reshape(gc.shape) != gc).sum())
            st['ncodes'] += gc.numel()
            V['S'][sl] = gc.view(V['S'][sl].shape)
            if 'SC' in V:
                gs = _tt(G['scales'][fi], device)
                st['sflips'] += int((V['SC'][sl].reshape(gs.shape) != gs).sum())
                V['SC'][sl] = gs.view(V['SC'][sl].shape)
        assert torch.equal(V['NPTR'][sl, :hv].cpu(), torch.full((B, hv), (n + 1) % m, dtype=torch.int32))
    assert len(folds) == T // m
    keep = torch.ones_like(raw, dtype=torch.bool)
    keep[1:B + 1, 64:64 + lay.nbytes] = False
    assert torch.equal(raw[keep], before[keep]), 'bytes outside the live slots were written'
    return st


def check_stats(name, st, o_tol=2e-5):
    print(f"\n[{name}] max rel |o - o_ref| {st['worst']:.2e}; buffer entries flipped {st['flips']}/{st['nbuf']}; "
          f"codes differing after folds {st['cflips']}/{st['ncodes']}; scales differing {st['sflips']}")
    assert st['worst'] < o_tol, st['worst']
    assert st['flips'] <= max(1, 1e-4 * st['nbuf']), st['flips']
    assert st['cflips'] <= max(1, 1e-4 * st['ncodes']), st['cflips']
    assert st['sflips'] <= max(1, 1e-4 * max(st['ncodes'], 1)), st['sflips']
