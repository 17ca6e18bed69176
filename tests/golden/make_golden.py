"""Generates the golden vectors under tests/golden/ by running the REFERENCE implementation's own torch classes
(``statequant.kernels.Reference{GDN,Mamba2,KDA}State``, ``pack_vk``, ``SlotLayout.read``) on the seeded cases of
``tests/cases.py``.

    python tests/golden/make_golden.py --reference /path/to/StateQuant/src

The reference is only needed here; the tests read the .npz files.  Each decode fixture holds, per step, the
reference's output, the buffer entry it appended (as stored: int8 codes + fp16 scale, or bf16 bits), the cumulative
decay, and after every fold the stored codes and scales.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.dont_write_bytecode = True
from cases import CASES, PACK_CASES, fmt_of, make_inputs, pack_input  # noqa: E402


def np_of(t):
    """torch -> numpy; bf16 as int16 bit patterns."""
    return t.view(torch.int16).numpy().copy() if t.dtype == torch.bfloat16 else t.numpy().copy()


def stored_entry(x, bb):
    """A buffered vector as the reference holds it (float, already rounded) -> its stored form."""
    if bb == 16:
        b = x.to(torch.bfloat16)
        assert torch.equal(b.float(), x)
        return b.view(torch.int16).numpy(), np.zeros(x.shape[:-1], np.float16)
    amax = x.abs().amax(-1, keepdim=True)
    s = (amax.clamp_min(1e-8) / 127).to(torch.float16).float().clamp_min(2. ** -24)
    s = torch.where(amax > 0, amax / 127, s)             # rounded rows have amax = 127 s exactly
    code = torch.round(x / s)
    assert torch.equal(code * s, x) and code.abs().max() <= 127
    assert torch.equal(s.to(torch.float16).float(), s)
    return code.to(torch.int8).numpy(), s.squeeze(-1).to(torch.float16).numpy()


def run_case(name, c, sq, K):
    inp = make_inputs(c)
    fmt = fmt_of(c, sq.Quantizer)
    B, hv, hk, dk, dv, m, bb, T = (c[k] for k in ('B', 'hv', 'hk', 'dk', 'dv', 'm', 'bb', 'T'))
    kind = c['kind']
    S0 = inp['S0']
    if kind == 'gdn':
        ref = K.ReferenceGDNState(S0.transpose(1, 2).contiguous(), fmt, m=m, hv=hv, hk=hk, buffer_bits=bb)
    elif kind == 'm2':
        ref = K.ReferenceMamba2State(S0, fmt, m=m, hv=hv, hk=hk, buffer_bits=bb)
    else:
        ref = K.ReferenceKDAState(S0, fmt, m=m, hv=hv, buffer_bits=bb)
    rec = dict(o=[], Kc=[], Ks=[], Uc=[], Us=[], G=[], fold_t=[], codes=[], scales=[])
    rec['codes0'], rec['scales0'] = np_of(ref.codes), (np_of(ref.scales) if ref.scales is not None else np.zeros(1))
    for t in range(T):
        n = ref.n
        if kind == 'gdn':
            o = ref.step(inp['q'][t].reshape(B * hk, dk), inp['k'][t].reshape(B * hk, dk), inp['v'][t].reshape(B * hv, dv),
                         inp['g'][t].reshape(-1), inp['beta'][t].reshape(-1), dk ** -0.5)
        elif kind == 'm2':
            sp = c.get('softplus', True)
            o = ref.step(inp['x'][t], inp['dt'][t], inp['Bm'][t], inp['Cm'][t], inp['A'], inp['D'],
                         inp['dt_bias'] if sp else None, dt_softplus=sp, dt_limit=(0., float('inf')))
        else:
            o = ref.step(inp['q'][t].reshape(B * hv, dk), inp['k'][t].reshape(B * hv, dk), inp['v'][t].reshape(B * hv, dv),
                         inp['g'][t].reshape(B * hv, dk), inp['beta'][t].reshape(-1), dk ** -0.5)
        rec['o'].append(o.reshape(B * hv, dv).numpy().copy())
        folded = ref.n == 0
        # after a fold the reference keeps the buffer contents; slot n still holds this step's entry
        kc, ks = stored_entry(ref.K[:, n].clone(), bb)
        uc, us = stored_entry(ref.U[:, n].clone(), bb)
        rec['Kc'].append(kc); rec['Ks'].append(ks); rec['Uc'].append(uc); rec['Us'].append(us)
        rec['G'].append(ref.G[:, n].numpy().copy())
        if folded:
            rec['fold_t'].append(t)
            rec['codes'].append(np_of(ref.codes))
            rec['scales'].append(np_of(ref.scales) if ref.scales is not None else np.zeros(1))
    out = {k: np.stack(v) if len(v) else np.zeros(0) for k, v in rec.items() if isinstance(v, list)}
    out['codes0'], out['scales0'] = rec['codes0'], rec['scales0']
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True, help='the src directory of a StateQuant checkout')
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import statequant as sq
    import statequant.kernels as K
    torch.set_num_threads(1)

    # ---- pack / unpack known answers (incl. all-zero groups, fp16-subnormal scales, ragged key groups) ----
    pk = {}
    for bits, axis, group, dk, dv in PACK_CASES:
        S = pack_input(bits, axis, group, dk, dv)
        q = sq.Quantizer(bits, axis, group)
        c, s = K.pack_vk(S, q)
        tag = f'b{bits}{axis}{group}_{dk}x{dv}'
        pk[tag + '_codes'] = c.numpy()
        pk[tag + '_scales'] = s.numpy()
        assert torch.equal(K.unpack_vk(c, s, q, dk).transpose(1, 2),
                           sq.Quantizer(bits, axis, group, scale_dtype='fp16').fake(S.transpose(1, 2)))
    np.savez_compressed(os.path.join(HERE, 'pack.npz'), **pk)

    # ---- decode runs ----
    for name, c in CASES.items():
        out = run_case(name, c, sq, K)
        fix = out
        np.savez_compressed(os.path.join(HERE, name + '.npz'), **fix)
        print(name, {k: v.shape for k, v in fix.items()})

    # ---- read(): stored state advanced across the pending buffer ----
    rd = {}
    for name in ('gdn_int4k32_m8_b8', 'kda_int4k32_m8_b8', 'm2_int8k32_m8_b8'):
        c = CASES[name]
        inp = make_inputs(c)
        fmt = fmt_of(c, sq.Quantizer)
        B, hv, hk, dk, dv, m, bb = (c[k] for k in ('B', 'hv', 'hk', 'dk', 'dv', 'm', 'bb'))
        if c['kind'] == 'gdn':
            ref = K.ReferenceGDNState(inp['S0'].transpose(1, 2).contiguous(), fmt, m=m, hv=hv, hk=hk, buffer_bits=bb)
            lay = K.SlotLayout(fmt, hv, hk, dk, dv, m=m, buffer_bits=bb)
        elif c['kind'] == 'm2':
            ref = K.ReferenceMamba2State(inp['S0'], fmt, m=m, hv=hv, hk=hk, buffer_bits=bb)
            lay = K.Mamba2SlotLayout(fmt, hv, hk, dk, dv, m=m, buffer_bits=bb)
        else:
            ref = K.ReferenceKDAState(inp['S0'], fmt, m=m, hv=hv, buffer_bits=bb)
            lay = K.KDASlotLayout(fmt, hv, dk, dv, m=m, buffer_bits=bb)
        for t in range(5):                                      # leaves n = 5 pending entries
            if c['kind'] == 'gdn':
                ref.step(inp['q'][t].reshape(B * hk, dk), inp['k'][t].reshape(B * hk, dk), inp['v'][t].reshape(B * hv, dv),
                         inp['g'][t].reshape(-1), inp['beta'][t].reshape(-1), dk ** -0.5)
            elif c['kind'] == 'm2':
                ref.step(inp['x'][t], inp['dt'][t], inp['Bm'][t], inp['Cm'][t], inp['A'], inp['D'], inp['dt_bias'],
                         dt_softplus=True, dt_limit=(0., float('inf')))
            else:
                ref.step(inp['q'][t].reshape(B * hv, dk), inp['k'][t].reshape(B * hv, dk), inp['v'][t].reshape(B * hv, dv),
                         inp['g'][t].reshape(B * hv, dk), inp['beta'][t].reshape(-1), dk ** -0.5)
        # move the reference state into a slot blob of the reference's own layout, then read() it
        blob = lay.alloc(B + 1, device='cpu')
        V = lay.views(blob)
        sl = torch.arange(1, B + 1)
        V['S'][sl] = ref.codes.view(B, *V['S'].shape[1:])
        V['SC'][sl] = ref.scales.view(B, *V['SC'].shape[1:])
        n = ref.n
        for i in range(n):
            kc, ks = stored_entry(ref.K[:, i].clone(), bb)
            uc, us = stored_entry(ref.U[:, i].clone(), bb)
            V['KB'][sl, :, i] = torch.from_numpy(kc).view(B, -1, dk)
            V['KBS'][sl, :, i] = torch.from_numpy(ks).view(B, -1)
            V['UB'][sl, :, i] = torch.from_numpy(uc).view(B, hv, dv)
            V['UBS'][sl, :, i] = torch.from_numpy(us).view(B, hv)
            V['GB'][sl, :, i] = ref.G[:, i].view(B, hv, *V['GB'].shape[3:])
        V['GCUR'][sl] = ref.gcur.view(B, *V['GCUR'].shape[1:])
        V['NPTR'][sl] = n
        rd[name + '_blob'] = blob[:2].numpy()                   # slot 0 (padding) and slot 1
        rd[name + '_read'] = lay.read(V, sl[:1]).numpy()
        # the reference's own state() (Mamba2 / KDA) agrees with read() up to summation order
        if hasattr(ref, 'state'):
            assert torch.allclose(ref.state().view_as(lay.read(V, sl)), lay.read(V, sl), rtol=1e-5, atol=1e-6)
    np.savez_compressed(os.path.join(HERE, 'read.npz'), **rd)
    print('done')


if __name__ == '__main__':
    main()
