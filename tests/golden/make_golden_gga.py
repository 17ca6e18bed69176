"""Golden vectors of the GGA / STEP path, from the REFERENCE's torch code run on CPU:

    python tests/golden/make_golden_gga.py --reference /path/to/StateQuant/src

  gga_fit.npz    ``statequant.step_quant.fit`` on seeded states for every width (2, 4, 6, 8, 16)
  gga_step_*.npz ``integrations.vllm_gga.GGALayout.step`` (the reference's fp32 emulation of Algorithm 1, its Triton fit
                 replaced by the torch ``fit`` it is checked against) stepped from the state a packed slot holds.

The reference has no CPU packer for the packed slot, so the packed master trajectory is advanced with this
repository's oracle (``oracle.gga_store`` / ``gga_step``); before every step the reference emulation receives the
slot's decoded state and the window as decoded by the REFERENCE's own ``GGAPacked.window``, and its output, new
state and new window are recorded.  The tests replay the same trajectory (protocol of the reference's
tests/test_gga_packed.py:58-94).
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.dont_write_bytecode = True
from cases import GGA_CASES, fit_input, gga_inputs, gga_plan  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True, help='the src directory of a StateQuant checkout')
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import statequant as sq
    from statequant.integrations.vllm_gga import GGALayout, GGAPacked as RefPacked
    from statequant.step_quant import fit as torch_fit
    from oracle import oracle
    from statequant_b200.kernels import GGAPacked, StepPlan
    torch.set_num_threads(1)

    class Emu(GGALayout):
        def _quant(self, S, layer):
            b, w, two, _ = self._plan(layer, S.device)
            return S if S.shape[0] == 0 else torch_fit(S.contiguous(), b, w, self.method.group)

    # ---- the fit ----
    fx = {}
    for D in (64,):
        bits, w = gga_plan(5, D, seed=3, widths=[2, 4, 6, 8, 16])
        x = fit_input(D)
        fx[f'y{D}'] = torch_fit(x, bits, w).numpy()
    np.savez_compressed(os.path.join(HERE, 'gga_fit.npz'), **fx)

    # ---- the step ----
    for name, c in GGA_CASES.items():
        hv, hk, D, m, pw, T, B = c['hv'], c['hk'], c['d'], c['m'], c['pw'], c['T'], c['B']
        bits, w = gga_plan(hv, D, seed=c['seed'], widths=c['widths'])
        meth = sq.GGA(4, pivots=1)
        meth.plan = {0: (bits, w)}
        meth.masks = {0: bits == 16}
        mine = GGAPacked(StepPlan({0: (bits, w)}), hv, hk, D, D, pw=pw, m=m)
        refp = RefPacked(meth, hv, hk, D, D, pw=pw, m=m)
        assert refp.nbytes == mine.nbytes and refp.QOFF == mine.QOFF and refp.tables[0][0] == mine.tables[0][0]
        em = Emu(meth, hv, hk, D, D, pw=pw, m=m)
        inp = gga_inputs(c)
        Vp = mine.views(mine.alloc(B + 2, 'cpu'))
        Ve = em.views(em.alloc(B + 2, 'cpu'))
        idx = torch.tensor(c['idx'], dtype=torch.int32)
        ok = idx > 0
        li = idx.long()
        oracle.gga_store(mine, Vp, idx[ok], inp['S0'], 0)
        rec = dict(o=[], O=[], P=[], V=[], n=[], keep=[])
        for t in range(T):
            Ve['O'][li[ok]] = oracle.gga_load(mine, Vp, idx[ok], 0).transpose(-1, -2)
            if pw:
                P, V, n = refp.window(Vp, idx[ok])                 # the reference's decoder on these bytes
                Ve['P'][li[ok]], Ve['V'][li[ok]] = P, V
                Ve['NQ'][li[ok]] = n[:, None].expand(-1, 4).to(torch.int32)
            q, k, v, a, b = (inp[x][t] for x in ('q', 'k', 'v', 'a', 'b'))
            oe = torch.empty(B, hv, D)
            em.step(Ve, idx, q, k, v, oe, D ** -0.5, gate=(a, b, inp['A_log'], inp['dt_bias']), layer=0)
            op = torch.empty(B, hv, D)
            oracle.gga_step(mine, Vp, idx, q, k, v, op, D ** -0.5, (a, b, inp['A_log'], inp['dt_bias']), 0)
            rec['o'].append(oe.numpy().copy())
            if t in c['keep']:
                rec['keep'].append(t)
                rec['O'].append(Ve['O'][li[ok]].transpose(-1, -2).numpy().copy())
                if pw:
                    rec['P'].append(Ve['P'][li[ok]].numpy().copy())
                    rec['V'].append(Ve['V'][li[ok]].numpy().copy())
                    rec['n'].append(Ve['NQ'][li[ok], 0].numpy().copy())
            err = ((op - oe).norm() / oe.norm()).item()
            assert err < 1e-5, (name, t, err)
        np.savez_compressed(os.path.join(HERE, name + '.npz'), **{k_: np.stack(v_) if len(v_) else np.zeros(0)
                                                                   for k_, v_ in rec.items()})
        print(name, 'ok')


if __name__ == '__main__':
    main()
