"""The CPU oracle against golden vectors produced by the reference implementation (tests/golden/make_golden.py).

Protocol of the decode cases (the reference's own, tests/test_kernels.py:74-134 there): the oracle is stepped on a
slot blob; after every step its output is compared with the reference's (relative to the row maximum), the entry it
appended to the buffer and the codes / scales it wrote at a fold are compared byte for byte, mismatches are counted
against the reference's thresholds (<= 1e-4 of entries: fp32 sums that associate differently can move a value
across a rounding boundary), and the golden entry is adopted so that one flip is counted once.
"""
import pytest
import torch

from cases import CASES, PACK_CASES, pack_input
from harness import check_stats, field_diff, fresh_blob, layout_of, load_golden, replay_vs_golden
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


@pytest.mark.parametrize('name', list(CASES))
def test_decode_matches_reference(name):
    check_stats(name, replay_vs_golden(name, CASES[name], oracle=oracle))


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
