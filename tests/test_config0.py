"""Configuration 0 of the benchmark as stated: one Gated DeltaNet layer at Qwen3.5-4B shapes (B 4, 16 key heads, 32 value
heads, d 128), fp32 seeded inputs, zero initial state, 256 FREE-RUNNING decode steps under pace4 with the 8-token int8
buffer; every 32nd output and the final packed state are compared with the record the reference's own
``ReferenceGDNState`` produced (tests/golden/make_golden_cfg0.py).

Free-running means nothing is re-synchronised: a rounding that falls on the other side of a tie in step t changes
every later step (one flipped int4 code moves a state entry by a seventh of its group's largest value, and fp16 scales
follow the smallest perturbation), so this is the drift figure, not the per-step parity bar (that one is
tests/test_step_gpu.py's re-sync protocol).  Until the first flip the outputs agree to 3e-7.  The figures are printed;
the bars below bound them: outputs within 5e-2 of the largest output, at most 5e-4 of the final codes differing, by
one step, at most 2e-2 of the fp16 scales differing.
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden'))
from make_golden_cfg0 import B, D, HK, HV, M, T, cfg0_inputs  # noqa: E402

import statequant_b200 as sq  # noqa: E402
from harness import nibble_steps  # noqa: E402
from oracle import oracle  # noqa: E402
from statequant_b200.kernels import SlotLayout  # noqa: E402

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'cfg0_pace4_256.npz')


def _run(device, step):
    """256 free-running steps from a zero state; returns (outputs of every 32nd step, final blob on the host, layout)."""
    lay = SlotLayout(sq.Quantizer(4, 'k', 64), HV, HK, D, D, m=M, buffer_bits=8)
    blob = torch.zeros(B + 1, lay.nbytes, dtype=torch.uint8, device=device)
    V = lay.views(blob)
    idx = torch.arange(1, B + 1, dtype=torch.int32, device=device)
    lay.write(V, idx, torch.zeros(B, HV, D, D, device=device))
    inp = {k: v.to(device) for k, v in cfg0_inputs().items()}
    outs = []
    for t in range(T):
        out = torch.empty(B, HV, D, device=device)
        step(lay, V, idx, inp['q'][t], inp['k'][t], inp['v'][t], out, D ** -0.5, g=inp['g'][t], beta=inp['beta'][t])
        if t % 32 == 31:
            outs.append(out.cpu().clone())
    return torch.stack(outs), blob.cpu(), lay


def _against_golden(outs, blob, lay, what):
    G = np.load(GOLD)
    want = torch.from_numpy(G['o'])
    rel = ((outs - want).abs().amax(dim=(1, 2, 3)) / want.abs().amax(dim=(1, 2, 3)))
    V = lay.views(blob)
    codes = V['S'][1:B + 1].reshape(B * HV, D, D // 2)
    scales = V['SC'][1:B + 1].reshape(B * HV, D, 2)
    gc, gs = torch.from_numpy(G['codes']), torch.from_numpy(G['scales']).view(torch.float16)
    ndiff, maxstep = nibble_steps(codes, gc)
    sdiff = int((scales.view(torch.int16) != gs.view(torch.int16)).sum())
    print(f'\n[config 0, {what} vs the reference, free-running] max rel |o - o_ref| per kept step '
          f'{[f"{x:.1e}" for x in rel.tolist()]}; final state: {ndiff}/{gc.numel() * 2} codes differ (largest by {maxstep} '
          f'step(s)), {sdiff}/{gs.numel()} scales differ; counters {int(V["NPTR"][1:B + 1, :HV].max())}')
    assert int(V['NPTR'][1:B + 1, :HV].max()) == 0 and float(V['GCUR'][1:B + 1].abs().max()) == 0.   # 256 = 32 folds
    return float(rel.max()), ndiff / (gc.numel() * 2), maxstep, sdiff / gs.numel()


def test_config0_oracle_free_running_matches_reference():
    outs, blob, lay = _run('cpu', lambda lay, *a, **k: oracle.gdn_step(lay, *a, **k))
    rel, cfrac, maxstep, sfrac = _against_golden(outs, blob, lay, 'oracle')
    assert rel < 5e-2 and cfrac < 5e-4 and maxstep <= 1 and sfrac < 2e-2


@pytest.mark.gpu
def test_config0_cuda_free_running():
    """CUDA free-running against the oracle free-running on the same inputs, and against the reference's record."""
    o_h, blob_h, lay = _run('cpu', lambda lay, *a, **k: oracle.gdn_step(lay, *a, **k))
    o_d, blob_d, _ = _run('cuda', lambda lay, *a, **k: lay.step(*a, **k))
    rel = float(((o_d - o_h).abs().amax(dim=(1, 2, 3)) / o_h.abs().amax(dim=(1, 2, 3))).max())
    Vh, Vd = lay.views(blob_h), lay.views(blob_d)
    nd, ms = nibble_steps(Vd['S'][1:B + 1], Vh['S'][1:B + 1])
    n = Vh['S'][1:B + 1].numel() * 2
    sd = int((Vd['SC'][1:B + 1].view(torch.int16) != Vh['SC'][1:B + 1].view(torch.int16)).sum())
    print(f'\n[config 0, CUDA vs oracle, free-running] max rel |o - o_oracle| {rel:.1e}; final state: {nd}/{n} codes differ '
          f'(largest by {ms} step(s)), {sd} scales differ')
    assert rel < 5e-2 and nd / n < 5e-4 and ms <= 1
    rel_g, cfrac, maxstep, sfrac = _against_golden(o_d, blob_d, lay, 'CUDA')
    assert rel_g < 5e-2 and cfrac < 5e-4 and maxstep <= 1 and sfrac < 2e-2
