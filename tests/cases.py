"""Seeded decode cases shared by the golden-vector generator and the parity tests.

Inputs come from ``numpy.random.RandomState`` (a frozen generator: the same bits on every machine), so a fixture
only has to hold what the reference computed from them.
"""
from __future__ import annotations

import numpy as np
import torch

# name -> kind, fmt (bits, axis, group) or 'bf16' / 'fp32', B sequences, heads, dims, buffer length, buffer bits, steps
CASES = {
    'gdn_int4k32_m8_b8':   dict(kind='gdn', fmt=(4, 'k', 32), B=2, hv=4, hk=2, dk=64, dv=64, m=8, bb=8, T=20, seed=11),
    'gdn_int8k32_m4_b16':  dict(kind='gdn', fmt=(8, 'k', 32), B=2, hv=4, hk=2, dk=64, dv=64, m=4, bb=16, T=13, seed=12),
    'gdn_int4v32_m8_b8':   dict(kind='gdn', fmt=(4, 'v', 32), B=2, hv=4, hk=2, dk=64, dv=64, m=8, bb=8, T=17, seed=13),
    'gdn_int8v32_m2_b8':   dict(kind='gdn', fmt=(8, 'v', 32), B=1, hv=4, hk=4, dk=64, dv=64, m=2, bb=8, T=7, seed=14),
    'gdn_bf16_m4_b8':      dict(kind='gdn', fmt='bf16', B=2, hv=2, hk=1, dk=64, dv=64, m=4, bb=8, T=9, seed=15),
    'gdn_pace4_qwen':      dict(kind='gdn', fmt=(4, 'k', 64), B=1, hv=4, hk=2, dk=128, dv=128, m=8, bb=8, T=17, seed=16),
    'gdn_int4k64_m1_b8':   dict(kind='gdn', fmt=(4, 'k', 64), B=1, hv=2, hk=2, dk=128, dv=128, m=1, bb=8, T=4, seed=17),
    # head dims that are not powers of two (reference: tests/test_kernels_nonpow2.py): idle lanes, a short last key group
    'gdn_int8k32_96x192':  dict(kind='gdn', fmt=(8, 'k', 32), B=1, hv=4, hk=2, dk=96, dv=192, m=4, bb=8, T=9, seed=18),
    'gdn_int4k64_96x64':   dict(kind='gdn', fmt=(4, 'k', 64), B=2, hv=2, hk=1, dk=96, dv=64, m=8, bb=8, T=17, seed=19),
    'gdn_int4v32_192x96':  dict(kind='gdn', fmt=(4, 'v', 32), B=1, hv=2, hk=2, dk=192, dv=96, m=2, bb=16, T=5, seed=20),
    'm2_int8k32_m8_b8':    dict(kind='m2', fmt=(8, 'k', 32), B=2, hv=4, hk=2, dk=128, dv=64, m=8, bb=8, T=18, seed=21),
    'm2_int4k64_m4_b16':   dict(kind='m2', fmt=(4, 'k', 64), B=2, hv=4, hk=1, dk=128, dv=64, m=4, bb=16, T=9, seed=22,
                                softplus=False),
    'm2_int4v16_m8_b8':    dict(kind='m2', fmt=(4, 'v', 16), B=1, hv=4, hk=2, dk=128, dv=64, m=8, bb=8, T=17, seed=23),
    'm2_bf16_m4_b8':       dict(kind='m2', fmt='bf16', B=1, hv=4, hk=2, dk=128, dv=64, m=4, bb=8, T=9, seed=24),
    'kda_int4k32_m8_b8':   dict(kind='kda', fmt=(4, 'k', 32), B=2, hv=4, hk=4, dk=64, dv=64, m=8, bb=8, T=18, seed=31),
    'kda_int8v32_m4_b16':  dict(kind='kda', fmt=(8, 'v', 32), B=1, hv=4, hk=4, dk=64, dv=64, m=4, bb=16, T=9, seed=32),
    'kda_pace4':           dict(kind='kda', fmt=(4, 'k', 64), B=1, hv=2, hk=2, dk=128, dv=128, m=8, bb=8, T=17, seed=33),
}


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def make_inputs(c):
    """All inputs of a case as fp32 torch tensors: initial states S0 (value-major [B*hv, dv, dk]) and per-step
    activations, stacked over T."""
    r = np.random.RandomState(c['seed'])
    B, hv, hk, dk, dv, T = c['B'], c['hv'], c['hk'], c['dk'], c['dv'], c['T']
    f = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))      # noqa: E731
    out = {'S0': f(r.standard_normal((B * hv, dv, dk)) * 0.5)}
    if c['kind'] == 'gdn':
        out['q'] = f(r.standard_normal((T, B, hk, dk)))
        out['k'] = f(r.standard_normal((T, B, hk, dk)))
        out['v'] = f(r.standard_normal((T, B, hv, dv)))
        out['g'] = f(np.log(sigmoid(r.standard_normal((T, B, hv)) + 2.0)))
        out['beta'] = f(sigmoid(r.standard_normal((T, B, hv))))
    elif c['kind'] == 'm2':
        out['x'] = f(r.standard_normal((T, B, hv, dv)))
        out['dt'] = f(r.standard_normal((T, B, hv)))
        if not c.get('softplus', True):                  # dt given directly: no transcendental before the decay
            out['dt'] = f(r.uniform(0.0, 0.15, (T, B, hv)))
        out['Bm'] = f(r.standard_normal((T, B, hk, dk)))
        out['Cm'] = f(r.standard_normal((T, B, hk, dk)))
        out['A'] = f(-np.exp(r.uniform(0.0, np.log(16.0), hv)))
        out['D'] = f(r.standard_normal(hv))
        out['dt_bias'] = f(r.uniform(-4.0, -2.0, hv))
    else:
        out['q'] = f(r.standard_normal((T, B, hv, dk)))
        out['k'] = f(r.standard_normal((T, B, hv, dk)))
        out['v'] = f(r.standard_normal((T, B, hv, dv)))
        out['g'] = f(np.log(sigmoid(r.standard_normal((T, B, hv, dk)) + 3.0)))
        out['beta'] = f(sigmoid(r.standard_normal((T, B, hv))))
    return out


def fmt_of(c, Quantizer):
    return c['fmt'] if isinstance(c['fmt'], str) else Quantizer(*c['fmt'])


# pack / unpack known-answer cases: (bits, axis, group, dk, dv); dk 96 has a ragged last key group
PACK_CASES = [(b, a, g, dk, dv) for b in (4, 8) for a in ('k', 'v') for g in (16, 32, 64)
              for dk, dv in ((64, 32), (96, 64)) if not (a == 'v' and dv % g)]


def pack_input(bits, axis, group, dk, dv):
    """fp32 [3, dv, dk] with all-zero groups (head 0) and scales in the fp16 subnormal range (head 1)."""
    r = np.random.RandomState(1000 + bits * 7 + group + dk + (axis == 'v'))
    S = torch.from_numpy((r.standard_normal((3, dv, dk)) * r.uniform(0, 3, (3, dv, 1))).astype(np.float32))
    S[0, :, :dk // 2] = 0
    S[1] *= 1e-6
    return S


# ---- GGA / STEP cases: per-head widths of one layer, window on / off; idx has a padding row -------------------
GGA_CASES = {
    'gga_step_pw':   dict(hv=4, hk=2, d=64, m=8, pw=True, T=11, B=2, idx=[0, 3], widths=[2, 4, 16, 8], seed=51,
                          keep=[0, 8, 10]),
    'gga_step_nopw': dict(hv=4, hk=2, d=64, m=8, pw=False, T=4, B=2, idx=[-1, 1], widths=[6, 4, 16, 2], seed=52,
                          keep=[0, 3]),
    'gga_step_128':  dict(hv=2, hk=2, d=128, m=4, pw=True, T=6, B=1, idx=[1], widths=[4, 6], seed=53, keep=[5]),
}


def gga_plan(hv, d, seed, widths):
    r = np.random.RandomState(seed)
    return torch.tensor(widths, dtype=torch.int64), torch.from_numpy((r.rand(hv, d) + 0.5).astype(np.float32))


def gga_inputs(c):
    r = np.random.RandomState(c['seed'] + 100)
    B, hv, hk, D, T = c['B'], c['hv'], c['hk'], c['d'], c['T']
    live = sum(1 for i in c['idx'] if i > 0)
    f = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))      # noqa: E731
    return dict(S0=f(r.standard_normal((live, hv, D, D)) * 0.3),                    # value-major [P, HV, dv, dk]
                q=f(r.standard_normal((T, B, hk, D))), k=f(r.standard_normal((T, B, hk, D))),
                v=f(r.standard_normal((T, B, hv, D))), a=f(r.standard_normal((T, B, hv)) * 0.5 - 2),
                b=f(r.standard_normal((T, B, hv))), A_log=f(r.standard_normal(hv) * 0.3),
                dt_bias=f(r.standard_normal(hv) * 0.3))


def fit_input(D):
    """States for the stand-alone fit: [2, 5, D, D] with columns spanning three decades."""
    r = np.random.RandomState(40 + D)
    return torch.from_numpy((r.standard_normal((2, 5, D, D)) * np.logspace(-3, 0, D)).astype(np.float32))
