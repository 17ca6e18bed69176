"""The CPU oracle against golden vectors produced by the reference implementation (tests/golden/make_golden.py).

Protocol of the decode cases (the reference's own, tests/test_kernels.py:74-134 there): the oracle is stepped on a
slot blob; after every step its output is compared with the reference's (relative to the row maximum), the entry it
appended to the buffer and the codes / scales it wrote at a fold are compared byte for byte, mismatches are counted
against the reference's thresholds (<= 1e-4 of entries: fp32 sums that associate differently can move a value
across a rounding boundary), and the golden entry is adopted so that one flip is counted once.
"""
import numpy as np
import pytest
import torch

from cases import CASES, PACK_CASES, make_inputs, pack_input
from harness import field_diff, fresh_blob, layout_of, load_golden, run_step, step_args
from oracle import oracle

import statequant_b200 as sq
from statequant_b200.kernels import pack_vk, unpack_vk


@pytest.mark.parametrize('bits,axis,group,dk,dv', PACK_CASES)
def test_pack_matches_reference(bits, axis, group, dk, dv):
    G = load_golden('pack')
    tag = f'b{bits}{axis}{group}_{dk}x{dv}'
    S = pack_input(bits, axis, group, dk, dv)
    want_c, want_s = torch.from_numpy(G[tag + '_codes']), torch.from_numpy(G[tag + '_scales'])
    # the package's torch packer (product, prefill side)
    c, s = pack_vk(S, sq.Quantizer(bits, axis, group))
    assert torch.equal(c, want_c) and torch.equal(s, want_s)
    # the oracle's C packer
    c2, s2 = oracle.pack_vk(S, bits, axis == 'k', group)
    assert torch.equal(c2, want_c) and torch.equal(s2.view_as(want_s), want_s)
    x = unpack_vk(c, s, sq.Quantizer(bits, axis, group), dk)
    assert torch.equal(oracle.unpack_vk(c, s, bits, axis == 'k', group, dk), x)
    assert torch.equal(x.transpose(1, 2), sq.Quantizer(bits, axis, group, scale_dtype='fp16').fake(S.transpose(1, 2)))


def _adopt_entry(c, lay, V, sl, n, G, t):
    B, hv, hk, dk, dv = c['B'], c['hv'], c['hk'], c['dk'], c['dv']
    kc, uc = torch.from_numpy(G['Kc'][t]), torch.from_numpy(G['Uc'][t])
    if c['bb'] == 16:
        kc, uc = kc.view(torch.bfloat16), uc.view(torch.bfloat16)
    V['KB'][sl, :, n] = kc.view(B, hk, dk)
    V['UB'][sl, :, n] = uc.view(B, hv, dv)
    if c['bb'] == 8:
        V['KBS'][sl, :, n] = torch.from_numpy(G['Ks'][t]).view(B, hk)
        V['UBS'][sl, :, n] = torch.from_numpy(G['Us'][t]).view(B, hv)


@pytest.mark.parametrize('name', list(CASES))
def test_decode_matches_reference(name):
    c = CASES[name]
    G = load_golden(name)
    inp = make_inputs(c)
    lay = layout_of(c)
    B, hv, hk, dk, dv, m, T = c['B'], c['hv'], c['hk'], c['dk'], c['dv'], c['m'], c['T']
    raw, blob = fresh_blob(lay, B + 2, seed=c['seed'], pad=64)
    V = lay.views(blob)
    sl = torch.arange(1, B + 1)
    lay.write(V, sl, inp['S0'].view(B, hv, dv, dk))
    codes0 = torch.from_numpy(G['codes0'])
    if codes0.dtype == torch.int16:
        codes0 = codes0.view(torch.bfloat16)
    assert torch.equal(V['S'][sl].reshape(codes0.shape), codes0)
    idx = torch.arange(1, B + 1, dtype=torch.int32)
    before = raw.clone()
    worst, flips, nbuf, cflips, ncodes, sflips = 0., 0, 0, 0, 0, 0
    folds = list(G['fold_t'])
    for t in range(T):
        n = int(V['NPTR'][1, 0])
        out = torch.full((B, hv, dv), 7.)
        run_step(c, lay, V, idx, step_args(c, inp, t), out, inp, oracle=oracle)
        want = torch.from_numpy(G['o'][t]).view(B, hv, dv)
        worst = max(worst, ((out - want).abs().max() / want.abs().max()).item())
        # the appended entry, as stored
        kc, uc = torch.from_numpy(G['Kc'][t]), torch.from_numpy(G['Uc'][t])
        if c['bb'] == 16:
            kc, uc = kc.view(torch.bfloat16), uc.view(torch.bfloat16)
        flips += int((V['KB'][sl, :, n].reshape(kc.shape) != kc).sum()) + int((V['UB'][sl, :, n].reshape(uc.shape) != uc).sum())
        nbuf += kc.numel() + uc.numel()
        if c['bb'] == 8:
            assert torch.equal(V['KBS'][sl, :, n].reshape(-1), torch.from_numpy(G['Ks'][t]).reshape(-1))
            sflips += int((V['UBS'][sl, :, n].reshape(-1) != torch.from_numpy(G['Us'][t]).reshape(-1)).sum())
        # cumulative decay: the same fp32 additions, bit for bit, unless the decay itself comes out of an in-kernel
        # softplus (libm's and torch's exp / log differ in the last place)
        gb, gw = V['GB'][sl, :, n].reshape(-1), torch.from_numpy(G['G'][t]).reshape(-1)
        if c['kind'] == 'm2' and c.get('softplus', True):
            assert torch.allclose(gb, gw, rtol=2e-6, atol=0), (gb - gw).abs().max()
            V['GB'][sl, :, n] = gw.view(V['GB'][sl, :, n].shape)
            if t not in folds:
                V['GCUR'][sl] = gw.view(V['GCUR'][sl].shape)
        else:
            assert torch.equal(gb, gw)
        _adopt_entry(c, lay, V, sl, n, G, t)
        if t in folds:
            fi = folds.index(t)
            assert int(V['NPTR'][1, 0]) == 0 and float(V['GCUR'][sl].abs().max()) == 0.
            gc = torch.from_numpy(G['codes'][fi])
            if gc.dtype == torch.int16:
                gc = gc.view(torch.bfloat16)
            cflips += int((V['S'][sl].reshape(gc.shape) != gc).sum())
            ncodes += gc.numel()
            V['S'][sl] = gc.view(V['S'][sl].shape)
            if 'SC' in V:
                gs = torch.from_numpy(G['scales'][fi])
                sflips += int((V['SC'][sl].reshape(gs.shape) != gs).sum())
                V['SC'][sl] = gs.view(V['SC'][sl].shape)
        else:
            assert int(V['NPTR'][1, 0]) == (n + 1) % m
        assert torch.equal(V['NPTR'][sl, :hv], torch.full((B, hv), (n + 1) % m, dtype=torch.int32))
    print(f'\n[{name}] max rel |o - o_ref| {worst:.2e}; buffer entries flipped {flips}/{nbuf}; codes differing after '
          f'folds {cflips}/{ncodes}; scales differing {sflips}')
    assert len(folds) == T // m
    assert worst < 2e-5, worst
    assert flips <= max(1, 1e-4 * nbuf), flips
    assert cflips <= max(1, 1e-4 * ncodes), cflips
    assert sflips <= max(1, 1e-4 * ncodes), sflips
    # nothing outside the live slots was written (slot 0, the spare slot, the padding around each slot)
    keep = torch.ones_like(raw, dtype=torch.bool)
    keep[1:B + 1, 64:64 + lay.nbytes] = False
    assert torch.equal(raw[keep], before[keep])


@pytest.mark.parametrize('name', ['gdn_int4k32_m8_b8', 'kda_int4k32_m8_b8', 'm2_int8k32_m8_b8'])
def test_read_matches_reference(name):
    """read(): the stored state advanced across its pending buffer, product torch path and oracle vs the reference."""
    c = CASES[name]
    G = load_golden('read')
    lay = layout_of(c)
    blob = torch.from_numpy(G[name + '_blob']).clone()
    V = lay.views(blob)
    want = torch.from_numpy(G[name + '_read'])
    got = lay.read(V, torch.tensor([1]))
    assert torch.allclose(got, want, rtol=1e-6, atol=1e-7), (got - want).abs().max()
    got2 = oracle.slot_read(lay, V, torch.tensor([1]))
    assert torch.allclose(got2, want, rtol=1e-5, atol=1e-6), (got2 - want).abs().max()


def test_write_roundtrip_and_reset():
    """write() stores pack_vk's bytes and empties the buffer; the oracle's writer produces the same bytes."""
    c = CASES['gdn_int4k32_m8_b8']
    lay = layout_of(c)
    raw, blob = fresh_blob(lay, 4, seed=3)
    blob2 = blob.clone()
    V, V2 = lay.views(blob), lay.views(blob2)
    S = torch.randn(2, c['hv'], c['dv'], c['dk'], generator=torch.Generator().manual_seed(1))
    idx = torch.tensor([3, 1])
    lay.write(V, idx, S)
    oracle.slot_write(lay, V2, idx, S)
    assert field_diff(lay, blob, blob2, [1, 3]) == {k: 0 for k in V} or \
        all(v == 0 for k, v in field_diff(lay, blob, blob2, [1, 3]).items() if k in ('S', 'SC', 'GCUR', 'NPTR'))
    cc, ss = pack_vk(S.reshape(-1, c['dv'], c['dk']), sq.Quantizer(*c['fmt']))
    assert torch.equal(lay.read(V, idx), unpack_vk(cc, ss, sq.Quantizer(*c['fmt']), c['dk']).view_as(S))
    assert V['NPTR'][idx, 0].tolist() == [0, 0] and float(V['GCUR'][idx].abs().max()) == 0.
