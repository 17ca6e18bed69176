"""Parity of the sm_100a decode step with the reference, on a B200: against the reference's golden vectors and
against the CPU oracle on the same blob bytes, through the C ABI (``layout.step`` -> ``sqb_*_step``)."""
import pytest
import torch

from cases import CASES, make_inputs
from harness import (check_stats, field_diff, fresh_blob, layout_of, replay_vs_golden, run_step, step_args)
from oracle import oracle

import statequant_b200 as sq
from statequant_b200.kernels import (KDASlotLayout, Mamba2SlotLayout, PackedGDNState, PackedKDAState,
                                     PackedMamba2State, SlotLayout)

pytestmark = pytest.mark.gpu
DEV = 'cuda'


@pytest.fixture(params=['fused', 'mma', 'staged', 'generic'])
def kernel_path(request):
    """Every device code path: the tensor-core kernels with the fold fused into the m-th token's launch (default
    wherever their shape conditions hold), the tensor-core step followed by the separate fold launch, the staged
    SIMT kernel with the fold launch, and the generic kernel, which folds inside its own launch.  A path that does
    not take a shape falls through to the next one."""
    from statequant_b200 import _cabi
    _cabi.set_option('kernel_path', {'generic': 1, 'staged': 2, 'mma': 3, 'fused': 4}[request.param])
    base = _cabi.device_status()
    yield request.param
    _cabi.set_option('kernel_path', 0)
    assert _cabi.device_status() == base, 'a bounded wait ran out on the device'


@pytest.mark.parametrize('name', list(CASES))
def test_decode_matches_reference_golden(name, kernel_path):
    """The CUDA step against the reference's golden record (re-sync protocol of the reference's own tests)."""
    check_stats(name, replay_vs_golden(name, CASES[name], oracle=None, device=DEV))


def _oracle_lockstep(c, T, act_dtype, seed_slots=7, gate=False):
    """Step the same blob through CUDA and through the oracle from identical pre-step bytes, every step; compare
    outputs and every blob field; continue from the CUDA blob.  Slots are a random subset with padding rows."""
    inp = make_inputs(dict(c, T=T))
    if c.get('extreme'):                                      # read-out vectors: all zero, tiny, huge, by step
        for key in (('Cm',) if c['kind'] == 'm2' else ('q', 'k')):
            for t in range(T):
                inp[key][t] *= (1.0, 0.0, 1e-30, 1e20)[t % 4]
    lay = layout_of(c)
    B, hv, hk, dk, dv, m = c['B'], c['hv'], c['hk'], c['dk'], c['dv'], c['m']
    n_slots = 9
    raw, blob = fresh_blob(lay, n_slots, seed=seed_slots, pad=32)
    Vh = lay.views(blob)
    gen = torch.Generator().manual_seed(seed_slots)
    live = (torch.randperm(n_slots - 1, generator=gen)[:B] + 1)
    lay.write(Vh, live, inp['S0'].view(B, hv, dv, dk))
    for s in live.tolist():                                   # sequences at different buffer positions
        Vh['NPTR'][s] = int(torch.randint(0, m, (1,), generator=gen))
        # their live buffer entries must be sane numbers (garbage may hold NaN patterns); dead ones stay garbage
        n = int(Vh['NPTR'][s, 0])
        Vh['GB'][s][:, :n] = -torch.rand(Vh['GB'][s][:, :n].shape, generator=gen) * 0.3
        Vh['GCUR'][s] = -torch.rand(Vh['GCUR'][s].shape, generator=gen) * 0.1 - 0.3
        if c['bb'] == 8:
            Vh['KBS'][s][:, :n] = (torch.rand(Vh['KBS'][s][:, :n].shape, generator=gen) * 0.01 + 1e-3).half()
            Vh['UBS'][s][:, :n] = (torch.rand(Vh['UBS'][s][:, :n].shape, generator=gen) * 0.02 + 1e-3).half()
        else:
            Vh['KB'][s][:, :n] = (torch.randn(Vh['KB'][s][:, :n].shape, generator=gen) * 0.1).bfloat16()
            Vh['UB'][s][:, :n] = (torch.randn(Vh['UB'][s][:, :n].shape, generator=gen)).bfloat16()
    rawd = raw.to(DEV)
    blobd = rawd[:, 32:32 + lay.nbytes]
    Vd = lay.views(blobd)
    rows = B + 2
    st = dict(worst=0., buf=0, nbuf=0, codes=0, ncodes=0, scal=0)
    for t in range(T):
        perm = torch.randperm(rows, generator=gen)
        idx_l = [0] * rows
        src = [None] * rows
        order = live[torch.randperm(B, generator=gen)].tolist()
        for j, r in enumerate(perm.tolist()):
            if j < B:
                idx_l[r], src[r] = order[j], j
            else:
                idx_l[r] = 0 if j == B else -1
        idx = torch.tensor(idx_l, dtype=torch.int32)
        a = step_args(c, inp, t, act_dtype)
        # scatter the B activations into the padded batch
        ap = {}
        for k_, v_ in a.items():
            full = torch.zeros(rows, *v_.shape[1:], dtype=v_.dtype)
            for r in range(rows):
                if src[r] is not None:
                    full[r] = v_[src[r]]
            ap[k_] = full
        odt = torch.float32 if act_dtype == torch.float32 else act_dtype
        out_h = torch.full((rows, hv, dv), 7., dtype=odt)
        out_d = torch.full((rows, hv, dv), 7., dtype=odt, device=DEV)
        pre = raw.clone()
        run_step(c, lay, Vh, idx, ap, out_h, inp, oracle=oracle)
        run_step(c, lay, Vd, idx.to(DEV), {k_: v_.to(DEV) for k_, v_ in ap.items()}, out_d, inp)
        got = rawd.cpu()
        o_d, o_h = out_d.cpu().float(), out_h.float()
        for r in range(rows):
            if src[r] is None:
                assert torch.equal(o_d[r], torch.zeros_like(o_d[r]))
        den = o_h.abs().max()
        st['worst'] = max(st['worst'], ((o_d - o_h).abs().max() / den).item())
        d = field_diff(lay, got[:, 32:32 + lay.nbytes], blob, live.tolist())
        st['buf'] += d['KB'] + d['UB']
        st['nbuf'] += B * (hk * dk + hv * dv)
        st['scal'] += d.get('KBS', 0) + d.get('UBS', 0) + d.get('SC', 0)
        st['codes'] += d['S']
        st['ncodes'] += B * hv * dv * dk
        assert d['NPTR'] == 0, d
        if not (c['kind'] == 'm2' and c.get('softplus', True)) and not gate:
            assert d['GB'] == 0 and d['GCUR'] == 0, d
        # everything outside the live slots is untouched on the device
        keep = torch.ones_like(raw, dtype=torch.bool)
        for s in live.tolist():
            keep[s, 32:32 + lay.nbytes] = False
        assert torch.equal(got[keep], pre[keep]), 'bytes outside live slots changed'
        raw.copy_(got)                                          # re-sync: continue from the device's bytes
    return st


@pytest.mark.parametrize('name', list(CASES))
@pytest.mark.parametrize('act', ['fp32', 'bf16'])
def test_step_matches_oracle_on_slots(name, act, kernel_path):
    c = CASES[name]
    act_dtype = torch.float32 if act == 'fp32' else torch.bfloat16
    st = _oracle_lockstep(c, T=2 * c['m'] + 3, act_dtype=act_dtype)
    print(f"\n[{name} {act}] max rel |o - o_oracle| {st['worst']:.2e}; buffer bytes differing {st['buf']}/{st['nbuf']}; "
          f"code bytes differing {st['codes']}/{st['ncodes']}; scales differing {st['scal']}")
    # bf16 outputs: both sides round the same fp32 value to bf16, so a last-place difference shows as one bf16 ulp
    assert st['worst'] < (2e-5 if act == 'fp32' else 1e-2), st['worst']
    assert st['buf'] <= max(1, 1e-4 * st['nbuf']), st
    assert st['codes'] <= max(1, 1e-4 * st['ncodes']), st
    assert st['scal'] <= max(1, 1e-4 * st['ncodes']), st


def test_gdn_in_kernel_gate_matches_oracle():
    c = dict(CASES['gdn_pace4_qwen'])
    inp = make_inputs(c)
    lay = layout_of(c)
    B, hv, hk, dk, dv = c['B'], c['hv'], c['hk'], c['dk'], c['dv']
    raw, blob = fresh_blob(lay, 4, seed=5)
    Vh = lay.views(blob)
    sl = torch.tensor([2])
    lay.write(Vh, sl, inp['S0'].view(B, hv, dv, dk))
    blobd = blob.to(DEV)
    Vd = lay.views(blobd)
    g = torch.Generator().manual_seed(9)
    A_log = torch.randn(hv, generator=g) * 0.5
    dt_bias = torch.randn(hv, generator=g).bfloat16()
    idx = torch.tensor([2], dtype=torch.int32)
    for t in range(10):
        a = torch.randn(B, hv, generator=g).bfloat16()
        bb = torch.randn(B, hv, generator=g).bfloat16()
        q, k, v = inp['q'][t].bfloat16(), inp['k'][t].bfloat16(), inp['v'][t].bfloat16()
        oh = torch.empty(B, hv, dv)
        od = torch.empty(B, hv, dv, device=DEV)
        oracle.gdn_step(lay, Vh, idx, q, k, v, oh, dk ** -0.5, gate=(a, bb, A_log, dt_bias))
        lay.step(Vd, idx.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), od, dk ** -0.5,
                 gate=(a.to(DEV), bb.to(DEV), A_log.to(DEV), dt_bias.to(DEV)))
        assert ((od.cpu() - oh).abs().max() / oh.abs().max()).item() < 2e-5
        d = field_diff(lay, blobd.cpu(), blob, [2])
        assert d['S'] + d['KB'] + d['UB'] <= 2, d
        blob.copy_(blobd.cpu())
    # and the gate path agrees with passing g, beta computed in torch (reference: tests/test_slots.py:153-171)
    gt = -A_log.exp() * torch.nn.functional.softplus(a.float() + dt_bias.float())
    bt = bb.float().sigmoid()
    b1, b2 = blobd.clone(), blobd.clone()
    o1, o2 = torch.empty(B, hv, dv, device=DEV), torch.empty(B, hv, dv, device=DEV)
    lay.step(lay.views(b1), idx.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), o1, dk ** -0.5, g=gt.to(DEV), beta=bt.to(DEV))
    lay.step(lay.views(b2), idx.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), o2, dk ** -0.5,
             gate=(a.to(DEV), bb.to(DEV), A_log.to(DEV), dt_bias.to(DEV)))
    assert torch.allclose(o1, o2, rtol=1e-5, atol=1e-5), (o1 - o2).abs().max()


@pytest.mark.parametrize('name', ['gdn_pace4_qwen', 'gdn_int4v32_m8_b8', 'm2_int8k32_m8_b8', 'kda_pace4'])
def test_lockstep_container_equals_slot_path(name):
    """PackedGDNState / PackedMamba2State / PackedKDAState (contiguous tables, identity slot map) give the same
    bytes as the slot layout stepping the same sequences."""
    c = CASES[name]
    inp = make_inputs(c)
    lay = layout_of(c)
    B, hv, hk, dk, dv, m = c['B'], c['hv'], c['hk'], c['dk'], c['dv'], c['m']
    fmt = sq.Quantizer(*c['fmt'])
    blob = lay.alloc(B + 1, DEV)
    V = lay.views(blob)
    sl = torch.arange(1, B + 1, device=DEV)
    S0 = inp['S0'].to(DEV)
    lay.write(V, sl, S0.view(B, hv, dv, dk))
    if c['kind'] == 'gdn':
        ker = PackedGDNState(S0.transpose(1, 2), fmt, m=m, hv=hv, hk=hk, buffer_bits=c['bb'], out_dtype=torch.float32)
    elif c['kind'] == 'm2':
        ker = PackedMamba2State(S0, fmt, m=m, hv=hv, hk=hk, buffer_bits=c['bb'], out_dtype=torch.float32)
    else:
        ker = PackedKDAState(S0, fmt, m=m, hv=hv, buffer_bits=c['bb'], out_dtype=torch.float32)
    assert torch.equal(ker.codes.view(B, *V['S'].shape[1:]), V['S'][sl])
    idx = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
    for t in range(c['T']):
        a = {k_: v_.to(DEV) for k_, v_ in step_args(c, inp, t).items()}
        out = torch.empty(B, hv, dv, device=DEV)
        run_step(c, lay, V, idx, a, out, inp)
        if c['kind'] == 'gdn':
            o = ker.step(a['q'].reshape(B * hk, dk), a['k'].reshape(B * hk, dk), a['v'].reshape(B * hv, dv),
                         a['g'].reshape(-1), a['beta'].reshape(-1), dk ** -0.5)
        elif c['kind'] == 'm2':
            o = ker.step(a['x'], a['dt'], a['B'], a['C'], inp['A'].to(DEV), inp['D'].to(DEV), inp['dt_bias'].to(DEV),
                         dt_softplus=True)
        else:
            o = ker.step(a['q'], a['k'], a['v'], a['g'], a['beta'], dk ** -0.5)
        assert torch.equal(o.reshape(B, hv, dv), out), t
        assert ker.n == int(V['NPTR'][1, 0]) == (t + 1) % m
    assert torch.equal(ker.codes.view(B, *V['S'].shape[1:]), V['S'][sl])
    assert torch.equal(ker.scales.view(B, *V['SC'].shape[1:]), V['SC'][sl])
    assert torch.equal(ker.UB.view(B, *V['UB'].shape[1:]), V['UB'][sl])
    assert torch.equal(ker.KB.view(B, *V['KB'].shape[1:]), V['KB'][sl])


def test_gdn_q_k_per_value_head():
    """q, k handed per value head [B * hv, d_k] (the lockstep container's other input form) equal the per-key-head
    form when the value heads of a group share them (reference: tests/test_kernels.py:137-150)."""
    c = CASES['gdn_pace4_qwen']
    inp = make_inputs(c)
    B, hv, hk, dk, dv = c['B'], c['hv'], c['hk'], c['dk'], c['dv']
    S0 = inp['S0'].to(DEV).transpose(1, 2)
    fmt = sq.Quantizer(*c['fmt'])
    a = PackedGDNState(S0, fmt, m=8, hv=hv, hk=hk, out_dtype=torch.float32)
    b = PackedGDNState(S0, fmt, m=8, hv=hv, hk=hk, out_dtype=torch.float32)
    for t in range(10):
        qh, kh = inp['q'][t].to(DEV).reshape(B * hk, dk), inp['k'][t].to(DEV).reshape(B * hk, dk)
        qf = qh.reshape(B, hk, 1, dk).expand(-1, -1, hv // hk, -1).reshape(B * hv, dk).contiguous()
        kf = kh.reshape(B, hk, 1, dk).expand(-1, -1, hv // hk, -1).reshape(B * hv, dk).contiguous()
        v, g, be = inp['v'][t].to(DEV).reshape(B * hv, dv), inp['g'][t].to(DEV).reshape(-1), inp['beta'][t].to(DEV).reshape(-1)
        oa = a.step(qf, kf, v, g, be, dk ** -0.5).clone()
        ob = b.step(qh, kh, v, g, be, dk ** -0.5).clone()
        # the two input forms take different device code paths (fp32 sums associate differently)
        assert ((oa - ob).abs().max() / ob.abs().max()).item() < 2e-5
    assert (a.codes != b.codes).sum().item() <= 1e-4 * a.codes.numel() + 1 and torch.equal(a.KB, b.KB)
    assert (a.UB != b.UB).sum().item() <= 2


@pytest.mark.parametrize('name', ['gdn_pace4_qwen', 'm2_int8k32_m8_b8', 'kda_pace4'])
def test_cuda_graph_replay_equals_eager(name):
    """One captured padded batch replayed with changing slot tables and inputs gives the bytes of eager launches
    (reference: tests/test_slots.py:174-207)."""
    c = CASES[name]
    inp = make_inputs(dict(c, T=24))
    lay = layout_of(c)
    B, hv, hk, dk, dv = c['B'], c['hv'], c['hk'], c['dk'], c['dv']
    n_slots, rows = 6, 4
    blob = lay.alloc(n_slots, DEV)
    V = lay.views(blob)
    g = torch.Generator().manual_seed(4)
    S = torch.randn(n_slots - 1, hv, dv, dk, generator=g).to(DEV) * 0.5
    lay.write(V, torch.arange(1, n_slots, device=DEV), S)
    blob_e = blob.clone()
    Ve = lay.views(blob_e)
    idx = torch.zeros(rows, dtype=torch.int32, device=DEV)
    a0 = step_args(c, inp, 0)
    stat = {k_: torch.zeros(rows, *v_.shape[1:], dtype=v_.dtype, device=DEV) for k_, v_ in a0.items()}
    out = torch.zeros(rows, hv, dv, device=DEV)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        run_step(c, lay, V, idx, stat, out, inp)               # all rows padding: nothing touched
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    assert torch.equal(blob, blob_e)
    G = torch.cuda.CUDAGraph()
    with torch.cuda.graph(G):
        run_step(c, lay, V, idx, stat, out, inp)
    tables = [[5, 2, 3, 0], [2, 0, 0, -1], [3, 5, 0, 0], [5, 3, 2, 1], [0, 0, 0, 0], [5, 0, 2, -1]] * 3
    for t, tab in enumerate(tables):
        idx.copy_(torch.tensor(tab, dtype=torch.int32))
        a = step_args(c, inp, t)
        for k_, v_ in a.items():
            reps = -(-rows // v_.shape[0])
            stat[k_].copy_(v_.repeat(reps, *([1] * (v_.dim() - 1)))[:rows])
        G.replay()
        oe = torch.zeros_like(out)
        run_step(c, lay, Ve, idx, stat, oe, inp)
        torch.cuda.synchronize()
        assert torch.equal(out, oe), t
    assert torch.equal(blob, blob_e)
    assert len({int(V['NPTR'][s_, 0]) for s_ in (1, 2, 3, 5)}) > 1        # counters diverged


def test_fp32_state_slot():
    """The unpacked fp32 slot ('fp32' format): write stores S exactly, the step folds in fp32, read() predicts the
    step after a fold (reference: tests/test_slots.py:219-251)."""
    hv, hk, D, m = 4, 2, 128, 4
    lay = SlotLayout('fp32', hv, hk, D, D, m=m, buffer_bits=8)
    blob = torch.randint(0, 256, (8, lay.nbytes), dtype=torch.uint8).to(DEV)
    V = lay.views(blob)
    idx = torch.tensor([5, 2], dtype=torch.int32, device=DEV)
    g0 = torch.Generator().manual_seed(2)
    S = (torch.randn(2, hv, D, D, generator=g0) * 0.5).to(DEV)
    lay.write(V, idx, S)
    assert torch.equal(V['S'][idx.long()], S)
    for t in range(2 * m + 1):
        q, k = (torch.randn(2, hk, D, generator=g0).to(DEV) for _ in range(2))
        v = torch.randn(2, hv, D, generator=g0).to(DEV)
        gg = (-torch.rand(2, hv, generator=g0) * 0.08).to(DEV)
        beta = torch.rand(2, hv, generator=g0).sigmoid().to(DEV)
        out = torch.empty(2, hv, D, device=DEV)
        if t == 2 * m:
            St = lay.read(V, idx)
            qn = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
            kn = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            qx, kx = qn.repeat_interleave(hv // hk, 1), kn.repeat_interleave(hv // hk, 1)
            a = gg.exp()[..., None]
            u = beta[..., None] * (v - a * torch.einsum('phvk,phk->phv', St, kx))
            o_pred = a * torch.einsum('phvk,phk->phv', St, qx) + (qx * kx).sum(-1, keepdim=True) * u
        lay.step(V, idx, q, k, v, out, D ** -0.5, g=gg, beta=beta)
        if t == 2 * m - 1:
            Sf = V['S'][idx.long()]
            assert int(V['NPTR'][5, 0]) == 0
            assert not torch.equal(Sf, Sf.bfloat16().float())
    assert ((out - o_pred).norm() / o_pred.norm()).item() < 1e-5


def test_full_batch_properties_qwen_shapes():
    """BASELINE-size batch (256 rows x 32 value heads, pace4): determinism, padding rows, a sample of rows against
    the oracle, and the fold period (all counters wrap together)."""
    hv, hk, D, m, B = 32, 16, 128, 8, 256
    lay = SlotLayout(sq.Quantizer(4, 'k', 64), hv, hk, D, D, m=m)
    g0 = torch.Generator().manual_seed(1)
    blob = lay.alloc(B + 1, DEV)
    V = lay.views(blob)
    S = torch.randn(B, hv, D, D, generator=g0) * 0.3
    lay.write(V, torch.arange(1, B + 1, device=DEV), S.to(DEV))
    idx = (torch.randperm(B, generator=g0) + 1).to(torch.int32)
    idx[::17] = 0
    idxd = idx.to(DEV)
    blob2 = blob.clone()
    V2 = lay.views(blob2)
    sample = [int(s) for s in idx[1:6] if s > 0]
    for t in range(m + 1):
        q, k = (torch.randn(B, hk, D, generator=g0).bfloat16() for _ in range(2))
        v = torch.randn(B, hv, D, generator=g0).bfloat16()
        a, b = (torch.randn(B, hv, generator=g0).bfloat16() for _ in range(2))
        A_log, dtb = torch.randn(hv, generator=g0) * 0.3, torch.randn(hv, generator=g0)
        out = torch.empty(B, hv, D, dtype=torch.bfloat16, device=DEV)
        out2 = torch.empty_like(out)
        args = [x.to(DEV) for x in (q, k, v)]
        gate = tuple(x.to(DEV) for x in (a, b, A_log, dtb))
        pre = blob[torch.tensor(sample, device=DEV)].cpu()
        lay.step(V, idxd, *args, out, D ** -0.5, gate=gate)
        lay.step(V2, idxd, *args, out2, D ** -0.5, gate=gate)
        assert torch.equal(out, out2) and torch.equal(blob, blob2)         # deterministic
        assert torch.equal(out[idxd <= 0], torch.zeros_like(out[idxd <= 0]))
        # oracle on the sampled slots from their pre-step bytes
        hb = torch.zeros(B + 1, lay.nbytes, dtype=torch.uint8)
        hb[torch.tensor(sample)] = pre
        rows = [int((idx == s).nonzero()[0]) for s in sample]
        oh = torch.empty(len(rows), hv, D, dtype=torch.bfloat16)
        oracle.gdn_step(lay, lay.views(hb), idx[rows].contiguous(), q[rows].contiguous(), k[rows].contiguous(),
                        v[rows].contiguous(), oh, D ** -0.5,
                        gate=(a[rows].contiguous(), b[rows].contiguous(), A_log, dtb))
        assert torch.allclose(out[rows].cpu().float(), oh.float(), rtol=1e-2, atol=1e-3)
        d = field_diff(lay, blob.cpu(), hb, sample)
        assert d['S'] <= 1e-4 * len(sample) * hv * D * D // 2 + 1 and d['UB'] + d['KB'] <= 2, d
    n = V['NPTR'][idxd[idxd > 0].long(), 0]
    assert int(n.min()) == int(n.max()) == (m + 1) % m


def test_bad_tensors_raise():
    lay = SlotLayout(sq.Quantizer(4, 'k', 64), 4, 2, 128, 128)
    blob = lay.alloc(3, DEV)
    V = lay.views(blob)
    q = torch.zeros(2, 2, 128, device=DEV)
    v = torch.zeros(2, 4, 128, device=DEV)
    out = torch.zeros(2, 4, 128, device=DEV)
    gb = torch.zeros(2, 4, device=DEV)
    with pytest.raises(AssertionError):
        lay.step(V, torch.tensor([1, 2], device=DEV), q, q, v, out, 1.0, g=gb, beta=gb)          # int64 idx
    with pytest.raises(TypeError):
        lay.step(V, torch.tensor([1, 2], dtype=torch.int32, device=DEV), q.double(), q.double(), v, out, 1.0, g=gb, beta=gb)
    with pytest.raises(AssertionError):
        lay.step(V, torch.tensor([1, 2], dtype=torch.int32, device=DEV), q, q, v, out.transpose(1, 2), 1.0, g=gb, beta=gb)
    with pytest.raises(RuntimeError, match='d_k 80'):               # rows of 40 bytes: not whole 16-byte chunks
        l2 = SlotLayout(sq.Quantizer(4, 'k', 64), 4, 2, 80, 128)
        b2 = l2.alloc(2, DEV)
        l2.step(l2.views(b2), torch.tensor([1], dtype=torch.int32, device=DEV), torch.zeros(1, 2, 80, device=DEV),
                torch.zeros(1, 2, 80, device=DEV), torch.zeros(1, 4, 128, device=DEV), torch.zeros(1, 4, 128, device=DEV),
                1.0, g=torch.zeros(1, 4, device=DEV), beta=torch.zeros(1, 4, device=DEV))


@pytest.mark.parametrize('kind,fmt', [('gdn', (4, 'k', 64)), ('gdn', (8, 'k', 32)), ('gdn', (4, 'v', 32)),
                                      ('gdn', (8, 'v', 32)), ('m2', (8, 'k', 32)), ('kda', (4, 'k', 64))])
def test_device_read_write_match_torch(kind, fmt):
    """The device-side prefill boundary: write packs byte for byte like the torch packer, read gives the state
    advanced across the pending buffer (reference: slots.py:210-252, kda.py:351-386)."""
    g0 = torch.Generator().manual_seed(5)
    q = sq.Quantizer(*fmt)
    if kind == 'gdn':
        lay = SlotLayout(q, 8, 4, 128, 128, m=8)
    elif kind == 'm2':
        lay = Mamba2SlotLayout(q, 8, 2, 128, 64, m=8)
    else:
        lay = KDASlotLayout(q, 4, 128, 128, m=8)
    hv, dk, dv = lay.HV, lay.DK, lay.DV
    P = 5
    blob = lay.alloc(P + 2, DEV)
    blob.random_(0, 255)                                   # garbage everywhere: write must leave a clean slot
    V = lay.views(blob)
    idx = torch.tensor([3, 1, 6, 2, 5], dtype=torch.int32, device=DEV)
    S = torch.randn(P, hv, dv, dk, generator=g0) * torch.rand(P, hv, dv, 1, generator=g0) * 0.5
    assert lay._device_io(V)
    lay.write(V, idx, S.to(DEV))
    hb = torch.zeros(P + 2, lay.nbytes, dtype=torch.uint8)
    Vh = lay.views(hb)
    lay.write(Vh, idx.cpu(), S)                            # the torch path on a host blob
    for f in ('S', 'SC', 'NPTR', 'GCUR'):
        assert torch.equal(V[f][idx.long()].cpu(), Vh[f][idx.long().cpu()]), f
    # a few decode steps on the device, reading after each: the device read-out against torch on the same bytes
    c = dict(kind=kind, fmt=fmt, B=P, hv=hv, hk=lay.HK, dk=dk, dv=dv, m=8, bb=8, T=5, seed=9)
    inp = make_inputs(c)
    for t in range(5):
        args = {k: v.to(DEV) for k, v in step_args(c, inp, t, torch.float32).items()}
        out_d = torch.empty(P, hv, dv, device=DEV)
        run_step(c, lay, V, idx, args, out_d, inp)
        got = lay.read(V, idx).cpu()
        want = lay.read(lay.views(blob.cpu()), idx.cpu())   # the torch path on the same bytes
        assert ((got - want).abs().max() / want.abs().max()).item() < 1e-5, t
    assert int(V['NPTR'][idx.long(), 0].max()) == 5         # reading leaves the slots alone


def _full_batch(lay, steps, make, run_dev, run_oracle, sample_n=4, hv=None, dv=None):
    """BASELINE-size batch through the device twice (determinism), padding rows, and a sample of rows against the
    oracle from their pre-step bytes, across one fold period."""
    B = 256
    g0 = torch.Generator().manual_seed(3)
    blob = lay.alloc(B + 1, DEV)
    V = lay.views(blob)
    lay.write(V, torch.arange(1, B + 1, device=DEV), (torch.randn(B, hv, dv, lay.DK, generator=g0) * 0.3).to(DEV))
    idx = (torch.randperm(B, generator=g0) + 1).to(torch.int32)
    idx[::19] = 0
    idxd = idx.to(DEV)
    blob2 = blob.clone()
    V2 = lay.views(blob2)
    sample = [int(s) for s in idx[1:1 + sample_n] if s > 0]
    rows = [int((idx == s).nonzero()[0]) for s in sample]
    for t in range(steps):
        inp = make(B, g0)
        out = torch.empty(B, hv, dv, dtype=torch.bfloat16, device=DEV)
        out2 = torch.empty_like(out)
        pre = blob[torch.tensor(sample, device=DEV)].cpu()
        dev_inp = [x.to(DEV) for x in inp]
        run_dev(V, idxd, dev_inp, out)
        run_dev(V2, idxd, dev_inp, out2)
        assert torch.equal(out, out2) and torch.equal(blob, blob2), t                   # deterministic
        assert torch.equal(out[idxd <= 0], torch.zeros_like(out[idxd <= 0]))
        hb = torch.zeros(B + 1, lay.nbytes, dtype=torch.uint8)
        hb[torch.tensor(sample)] = pre
        oh = torch.empty(len(rows), hv, dv, dtype=torch.bfloat16)
        run_oracle(lay.views(hb), idx[rows].contiguous(), [x[rows].contiguous() for x in inp], oh)
        assert torch.allclose(out[rows].cpu().float(), oh.float(), rtol=1e-2, atol=1e-3), t
        d = field_diff(lay, blob.cpu(), hb, sample)
        assert d['S'] <= 1e-4 * len(sample) * hv * dv * lay.DK + 1 and d['UB'] + d['KB'] <= 4, (t, d)
    n = V['NPTR'][idxd[idxd > 0].long(), 0]
    assert int(n.min()) == int(n.max()) == steps % lay.m


def test_full_batch_properties_mamba2_shapes():
    """Nemotron-H shapes (128 heads in 8 groups, head_dim 64, d_state 128), batch 256, int8 k g32."""
    H, GR, DS, HD = 128, 8, 128, 64
    lay = Mamba2SlotLayout(sq.Quantizer(8, 'k', 32), H, GR, DS, HD, m=8)
    g1 = torch.Generator().manual_seed(8)
    A = -torch.exp(torch.rand(H, generator=g1) * 2.77)
    D = torch.randn(H, generator=g1)
    dtb = torch.rand(H, generator=g1) * 2.0 - 4.0
    Ad, Dd, dtbd = A.to(DEV), D.to(DEV), dtb.to(DEV)

    def make(B, g):
        f = lambda *s: torch.randn(*s, generator=g)                                      # noqa: E731
        return [f(B, H, HD).bfloat16(), f(B, H).bfloat16(), f(B, GR, DS).bfloat16(), f(B, GR, DS).bfloat16()]

    _full_batch(lay, 9, make,
                lambda V, i, x, o: lay.step(V, i, x[0], x[1], x[2], x[3], o, Ad, D=Dd, dt_bias=dtbd),
                lambda V, i, x, o: oracle.mamba2_step(lay, V, i, x[0], x[1], x[2], x[3], o, A, D, dtb),
                sample_n=2, hv=H, dv=HD)


def test_full_batch_properties_kda_shapes():
    """Kimi-Linear-like shapes (32 heads, d 128, per-channel decays), batch 256, pace4 state."""
    H, Dm = 32, 128
    lay = KDASlotLayout(sq.Quantizer(4, 'k', 64), H, Dm, Dm, m=8)

    def make(B, g):
        f = lambda *s: torch.randn(*s, generator=g)                                      # noqa: E731
        q, k = f(B, H, Dm), f(B, H, Dm)
        return [(q / q.norm(dim=-1, keepdim=True)).bfloat16(), (k / k.norm(dim=-1, keepdim=True)).bfloat16(),
                f(B, H, Dm).bfloat16(), torch.nn.functional.logsigmoid(f(B, H, Dm) + 3.0), torch.sigmoid(f(B, H))]

    _full_batch(lay, 9, make,
                lambda V, i, x, o: lay.step(V, i, x[0], x[1], x[2], x[3], x[4], o, Dm ** -0.5),
                lambda V, i, x, o: oracle.kda_step(lay, V, i, x[0], x[1], x[2], x[3], x[4], o, Dm ** -0.5),
                sample_n=3, hv=H, dv=Dm)


@pytest.mark.gpu
def test_two_devices_in_one_process():
    """The same decode run on two GPUs from one process (each under its own device guard) gives identical bytes:
    the kernels' shared-memory limits are per-device settings and are made on the device each launch runs on.
    Nine tokens, so that one fold launch (more than 48 KB of shared memory per CTA) runs on both."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    import statequant_b200 as sq
    from statequant_b200.kernels import SlotLayout
    lay = SlotLayout(sq.Quantizer(8, 'k', 32), 32, 16, 128, 128, m=8)
    g = torch.Generator().manual_seed(3)
    B = 8
    steps = [(torch.randn(B, 16, 128, generator=g).bfloat16(), torch.randn(B, 16, 128, generator=g).bfloat16(),
              torch.randn(B, 32, 128, generator=g).bfloat16(), torch.nn.functional.logsigmoid(torch.randn(B, 32, generator=g) + 2),
              torch.sigmoid(torch.randn(B, 32, generator=g))) for _ in range(9)]
    idx = torch.arange(1, B + 1, dtype=torch.int32)
    res = []
    for d in (0, 1):
        dev = torch.device('cuda', d)
        with torch.cuda.device(dev):
            blob = lay.alloc(B + 1, dev)
            views = lay.views(blob)
            out = torch.empty(B, 32, 128, dtype=torch.bfloat16, device=dev)
            outs = []
            for q, k, v, gg, bt in steps:
                lay.step(views, idx.to(dev), q.to(dev), k.to(dev), v.to(dev), out, 128 ** -0.5, g=gg.to(dev), beta=bt.to(dev))
                outs.append(out.cpu().clone())
            torch.cuda.synchronize(dev)
            res.append((blob.cpu(), outs))
    assert torch.equal(res[0][0], res[1][0])
    assert all(torch.equal(a, b) for a, b in zip(res[0][1], res[1][1]))
    assert res[0][0].any()


LONG_TAIL = [
    dict(kind='gdn', fmt=(8, 'k', 32), B=2, hv=4, hk=2, dk=128, dv=192, m=8, bb=8, seed=41),
    dict(kind='gdn', fmt=(4, 'k', 64), B=2, hv=4, hk=2, dk=128, dv=192, m=8, bb=8, seed=42),
    dict(kind='gdn', fmt=(4, 'v', 32), B=2, hv=4, hk=2, dk=128, dv=192, m=8, bb=8, seed=43),
    dict(kind='gdn', fmt=(4, 'k', 32), B=2, hv=4, hk=2, dk=64, dv=160, m=8, bb=16, seed=45),
    dict(kind='gdn', fmt=(8, 'k', 64), B=2, hv=4, hk=2, dk=192, dv=96, m=8, bb=8, seed=51),
    dict(kind='gdn', fmt='bf16', B=1, hv=2, hk=1, dk=96, dv=64, m=4, bb=8, seed=54),
    dict(kind='m2', fmt=(8, 'k', 32), B=2, hv=4, hk=2, dk=128, dv=96, m=8, bb=8, seed=46),
    dict(kind='m2', fmt=(8, 'k', 32), B=2, hv=4, hk=2, dk=96, dv=64, m=8, bb=8, seed=52),
    dict(kind='m2', fmt=(8, 'k', 32), B=2, hv=4, hk=2, dk=128, dv=80, m=8, bb=8, seed=56),   # head_dim 80
    dict(kind='m2', fmt=(4, 'k', 32), B=1, hv=4, hk=1, dk=96, dv=96, m=4, bb=16, seed=55),   # Mamba2: no short groups
    # long buffers (the reference allows m up to 32)
    dict(kind='gdn', fmt=(8, 'k', 32), B=2, hv=4, hk=2, dk=128, dv=128, m=16, bb=8, seed=61),
    dict(kind='gdn', fmt=(4, 'k', 64), B=1, hv=4, hk=2, dk=128, dv=128, m=32, bb=8, seed=62),
    dict(kind='m2', fmt=(8, 'k', 32), B=1, hv=4, hk=2, dk=128, dv=64, m=32, bb=8, seed=64),
    dict(kind='kda', fmt=(4, 'k', 64), B=1, hv=2, hk=2, dk=128, dv=128, m=16, bb=8, seed=66),
    dict(kind='gdn', fmt=(8, 'k', 32), B=1, hv=4, hk=2, dk=96, dv=192, m=16, bb=8, seed=68),
    # the fold launch's shared-memory plan does not fit: the whole step must fall to the generic kernel BEFORE anything
    # is appended (a step kernel that ran ahead of a refused fold would leave the slot between two states)
    dict(kind='gdn', fmt=(8, 'k', 32), B=1, hv=2, hk=1, dk=128, dv=512, m=32, bb=8, seed=69),
    # 4-bit codes scaled along v at the tensor-core kernel's shapes (per-warp scale-folded read-out vectors, the fold with
    # in-warp column maxima), fp32 and bf16 buffers
    dict(kind='gdn', fmt=(4, 'v', 32), B=2, hv=4, hk=2, dk=128, dv=128, m=8, bb=8, seed=71),
    dict(kind='gdn', fmt=(4, 'v', 32), B=1, hv=6, hk=2, dk=128, dv=128, m=8, bb=8, seed=72),
    dict(kind='gdn', fmt=(8, 'v', 32), B=2, hv=4, hk=2, dk=128, dv=128, m=8, bb=8, seed=78),   # pieces of four rows
    # key groups for which the tensor-core kernel folds in fp32 (more than one scale group, or less than one, per span)
    dict(kind='gdn', fmt=(8, 'k', 64), B=1, hv=4, hk=2, dk=128, dv=128, m=8, bb=8, seed=74),
    dict(kind='gdn', fmt=(4, 'k', 32), B=1, hv=4, hk=2, dk=128, dv=128, m=8, bb=8, seed=75),
    dict(kind='gdn', fmt=(4, 'k', 128), B=1, hv=4, hk=2, dk=128, dv=128, m=8, bb=8, seed=76),
    dict(kind='m2', fmt=(8, 'k', 128), B=1, hv=8, hk=2, dk=128, dv=64, m=8, bb=8, seed=77),
]


@pytest.mark.parametrize('c', LONG_TAIL, ids=lambda c: f"{c['kind']}-{c['fmt']}-{c['dk']}x{c['dv']}-m{c['m']}")
def test_long_tail_shapes_match_oracle(c, kernel_path):
    """Head dims that are not powers of two (the reference covers them in tests/test_kernels_nonpow2.py and
    docs/kernels.md:90-93): d_v 96 / 160 / 192 with the staged kernels, d_k 96 / 192 (idle lanes, a short last key
    group) with the generic one; and buffers of 16 and 32 entries.  Same bar as the other cases."""
    st = _oracle_lockstep(c, T=2 * c['m'] + 3, act_dtype=torch.float32)
    assert st['worst'] < 2e-5, st
    assert st['buf'] <= max(1, 1e-4 * st['nbuf']), st
    assert st['codes'] <= max(1, 1e-4 * st['ncodes']), st
    assert st['scal'] <= max(1, 1e-4 * st['ncodes']), st


INT4V_128 = dict(kind='gdn', fmt=(4, 'v', 32), B=1, hv=4, hk=2, dk=128, dv=128, m=8, bb=8, T=17, seed=73)


@pytest.mark.parametrize('name', ['gdn_pace4_qwen', 'm2_int8k32_m8_b8', 'kda_pace4', 'gdn_int4v_128', 'gdn_int8v_128'])
def test_extreme_read_out_vectors(name, kernel_path):
    """Read-out vectors that are all zero, tiny (1e-30) or huge (1e20) on alternating steps: the staged kernels hold
    them as fixed point with a per-vector power-of-two scale, which must cover the whole float range."""
    c = dict(INT4V_128 if name == 'gdn_int4v_128' else dict(INT4V_128, fmt=(8, 'v', 32), seed=79) if name == 'gdn_int8v_128'
             else CASES[name], extreme=True)
    st = _oracle_lockstep(c, T=2 * c['m'] + 3, act_dtype=torch.float32)
    assert st['worst'] < 2e-5, st
    assert st['buf'] <= max(1, 1e-4 * st['nbuf']), st
    assert st['codes'] <= max(1, 1e-4 * st['ncodes']), st


@pytest.mark.parametrize('preset,fmt', [('int8k', (8, 'k', 32)), ('int4v', (4, 'v', 32)), ('int8v', (8, 'v', 32))])
def test_full_batch_properties_gdn_presets(preset, fmt):
    """The benchmark's headline preset (int8k) and its int4v variant at the benchmark's shapes (32 value heads, 16 key
    heads, d 128, batch 256, bf16 activations, in-kernel gate): determinism, padding rows, a sample of rows against the
    oracle from their pre-step bytes, across one fold period."""
    hv, hk, D = 32, 16, 128
    lay = SlotLayout(sq.Quantizer(*fmt), hv, hk, D, D, m=8)
    g1 = torch.Generator().manual_seed(17)
    A_log, dtb = torch.randn(hv, generator=g1) * 0.3, torch.randn(hv, generator=g1)
    A_logd, dtbd = A_log.to(DEV), dtb.to(DEV)

    def make(B, g):
        f = lambda *s: torch.randn(*s, generator=g)                                      # noqa: E731
        return [f(B, hk, D).bfloat16(), f(B, hk, D).bfloat16(), f(B, hv, D).bfloat16(), (f(B, hv) + 2.0).bfloat16(),
                f(B, hv).bfloat16()]

    _full_batch(lay, 9, make,
                lambda V, i, x, o: lay.step(V, i, x[0], x[1], x[2], o, D ** -0.5, gate=(x[3], x[4], A_logd, dtbd)),
                lambda V, i, x, o: oracle.gdn_step(lay, V, i, x[0], x[1], x[2], o, D ** -0.5, gate=(x[3], x[4], A_log, dtb)),
                sample_n=3, hv=hv, dv=D)


def _hand_built_gdn_inputs(idx, q, k, v, out, scale, g, beta):
    """``sqb_gdn_inputs_t`` filled in by the test itself, field by field from the tensors' own pointers and strides
    (not by the package's marshalling code), for the oracle side of the strided-input check."""
    from statequant_b200 import _cabi
    code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
    a = _cabi.GdnInputs()
    a.idx = idx.data_ptr()
    a.q, a.sq = q.data_ptr(), q.stride(0) * q.element_size()
    a.k, a.sk = k.data_ptr(), k.stride(0) * k.element_size()
    a.v, a.sv = v.data_ptr(), v.stride(0) * v.element_size()
    a.g, a.sg = g.data_ptr(), g.stride(0) * g.element_size()
    a.beta, a.sbeta = beta.data_ptr(), beta.stride(0) * beta.element_size()
    a.out, a.so = out.data_ptr(), out.stride(0) * out.element_size()
    a.scale, a.rows, a.qk_per_key_head, a.gate = float(scale), out.shape[0], 1, 0
    a.qk_dtype, a.v_dtype, a.gb_dtype, a.out_dtype = code[q.dtype], code[v.dtype], code[g.dtype], code[out.dtype]
    return a


@pytest.mark.parametrize('name', ['gdn_pace4_qwen', 'gdn_int4k32_m8_b8'])
def test_strided_inputs_replay_reference_golden(name, kernel_path):
    """vLLM-style inputs: q, k, v are column slices of ONE [rows, 2 hk dk + hv dv] tensor (the conv output), g and beta
    column slices of one [rows, 2 hv] tensor, with padding rows in between (reference: tests/test_slots.py:174-207,
    integrations/vllm_plugin.py:395-397).  The CUDA step on them replays the reference's golden record; the oracle is
    stepped on the same strided host tensors through an argument struct the test fills in itself."""
    import ctypes as C
    from harness import load_golden
    c = CASES[name]
    G = load_golden(name)
    inp = make_inputs(c)
    lay = layout_of(c)
    B, hv, hk, dk, dv, m, T = c['B'], c['hv'], c['hk'], c['dk'], c['dv'], c['m'], c['T']
    rows = B + 2                                            # a padding row before and after
    blob_h = torch.zeros(B + 2, lay.nbytes, dtype=torch.uint8)
    sl = torch.arange(1, B + 1)
    lay.write(lay.views(blob_h), sl, inp['S0'].view(B, hv, dv, dk))
    blob_d = blob_h.to(DEV)
    Vh, Vd = lay.views(blob_h), lay.views(blob_d)
    idx = torch.tensor([0] + list(range(1, B + 1)) + [-1], dtype=torch.int32)
    worst = 0.
    for t in range(T):
        mixed = torch.zeros(rows, 2 * hk * dk + hv * dv)
        mixed[1:B + 1, :hk * dk] = inp['q'][t].reshape(B, -1)
        mixed[1:B + 1, hk * dk:2 * hk * dk] = inp['k'][t].reshape(B, -1)
        mixed[1:B + 1, 2 * hk * dk:] = inp['v'][t].reshape(B, -1)
        gb = torch.zeros(rows, 2 * hv)
        gb[1:B + 1, :hv], gb[1:B + 1, hv:] = inp['g'][t], inp['beta'][t]
        outs = []
        for dev, V in ((DEV, Vd), ('cpu', Vh)):
            mx, gx = mixed.to(dev), gb.to(dev)
            q = mx[:, :hk * dk].unflatten(-1, (hk, dk))
            k = mx[:, hk * dk:2 * hk * dk].unflatten(-1, (hk, dk))
            v = mx[:, 2 * hk * dk:].unflatten(-1, (hv, dv))
            g, beta = gx[:, :hv], gx[:, hv:]
            assert not q.is_contiguous() and not g.is_contiguous()
            out = torch.full((rows, hv, dv), 7., device=dev)
            if dev == 'cpu':
                a = _hand_built_gdn_inputs(idx, q, k, v, out, dk ** -0.5, g, beta)
                assert oracle.lib().sqo_gdn_step(C.byref(lay._struct(V)), C.byref(a)) == 0
            else:
                lay.step(V, idx.to(dev), q, k, v, out, dk ** -0.5, g=g, beta=beta)
            outs.append(out.cpu())
        want = torch.from_numpy(G['o'][t]).view(B, hv, dv)
        for o in outs:
            assert torch.equal(o[0], torch.zeros(hv, dv)) and torch.equal(o[-1], torch.zeros(hv, dv))
            worst = max(worst, ((o[1:B + 1] - want).abs().max() / want.abs().max()).item())
        d = field_diff(lay, blob_d.cpu(), blob_h, sl.tolist())
        assert d['NPTR'] == 0 and d['GB'] == 0 and d['S'] + d['KB'] + d['UB'] <= 2, (t, d)
        blob_h.copy_(blob_d.cpu())                           # re-sync on the device's bytes
    assert worst < 2e-5, worst


def test_bounded_wait_runs_out_and_is_reported():
    """The device-side waits for bulk copies are bounded: with a stage barrier made to expect more bytes than are ever
    copied (a test switch of the library; nothing faults, the copies themselves complete) and the bound shortened to
    a few milliseconds, every CTA gives up, the call returns, the health word counts the CTAs, the outputs of the
    rows are zeroed, and the slots' state is left as it was.  Afterwards the library works as before."""
    from statequant_b200 import _cabi
    hv, hk, D, B = 4, 2, 128, 3
    lay = SlotLayout(sq.Quantizer(8, 'k', 32), hv, hk, D, D, m=8)
    g0 = torch.Generator().manual_seed(21)
    blob = lay.alloc(B + 1, DEV)
    V = lay.views(blob)
    idx = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
    lay.write(V, idx, (torch.randn(B, hv, D, D, generator=g0) * 0.3).to(DEV))
    q, k = (torch.randn(B, hk, D, generator=g0).to(DEV) for _ in range(2))
    v = torch.randn(B, hv, D, generator=g0).to(DEV)
    gg = (-torch.rand(B, hv, generator=g0) * 0.1).to(DEV)
    beta = torch.rand(B, hv, generator=g0).to(DEV)
    out = torch.full((B, hv, D), 7., device=DEV)
    lay.step(V, idx, q, k, v, out, D ** -0.5, g=gg, beta=beta)               # a healthy step first
    torch.cuda.synchronize()
    base = _cabi.device_status()
    before = blob.clone()
    _cabi.set_option('kernel_path', 4)
    _cabi.set_option('wait_limit_us', 2000)
    _cabi.set_option('test_extra_tx', 64)
    try:
        out.fill_(7.)
        lay.step(V, idx, q, k, v, out, D ** -0.5, g=gg, beta=beta)
        torch.cuda.synchronize()
        assert _cabi.device_status() - base == B * hk                    # one count per CTA
        assert torch.equal(out, torch.zeros_like(out))
        d = field_diff(lay, blob.cpu(), before.cpu(), list(range(1, B + 1)))
        assert d['S'] == 0 and d['SC'] == 0 and d['UB'] == 0 and d['NPTR'] == 0 and d['GCUR'] == 0, d
    finally:
        _cabi.set_option('test_extra_tx', 0)
        _cabi.set_option('wait_limit_us', 1000000)
        _cabi.set_option('kernel_path', 0)
    blob.copy_(before)
    o2 = torch.empty_like(out)
    lay.step(V, idx, q, k, v, o2, D ** -0.5, g=gg, beta=beta)
    torch.cuda.synchronize()
    assert _cabi.device_status() - base == B * hk and torch.isfinite(o2).all() and o2.abs().max() > 0
