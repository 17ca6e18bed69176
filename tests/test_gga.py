"""GGA / STEP mixed-bit state with the pure-write window: the oracle against golden vectors of the reference's torch
code (CPU), and the CUDA kernels against the oracle on the same slot bytes and against the golden record (GPU)."""
import pytest
import torch

from cases import GGA_CASES, fit_input, gga_inputs, gga_plan
from harness import load_golden
from oracle import oracle

from statequant_b200.kernels import GGAPacked, StepPlan, head_bytes
from statequant_b200.kernels.gga import fit

DEV = 'cuda'


def _setup(c, device='cpu'):
    bits, w = gga_plan(c['hv'], c['d'], seed=c['seed'], widths=c['widths'])
    pk = GGAPacked(StepPlan({0: (bits, w)}), c['hv'], c['hk'], c['d'], c['d'], pw=c['pw'], m=c['m'])
    g = torch.Generator().manual_seed(c['seed'])
    blob = torch.randint(0, 256, (c['B'] + 2, pk.nbytes + 64), dtype=torch.uint8, generator=g)[:, :pk.nbytes]
    blob[:, :16] = 0                                             # counters of unused slots: sane
    return pk, bits, w, blob.to(device) if device != 'cpu' else blob


def test_fit_matches_reference():
    """The oracle's fit equals ``statequant.step_quant.fit`` bit for bit on every width."""
    G = load_golden('gga_fit')
    bits, w = gga_plan(5, 64, seed=3, widths=[2, 4, 6, 8, 16])
    y = oracle.stepquant_fit(fit_input(64), bits, w)
    assert torch.equal(y, torch.from_numpy(G['y64']))


def test_layout_accounting():
    """Slot offsets and sizes (reference: vllm_gga.py:169-205, docs: a 4-bit layer of 32 heads at 128 x 128 takes
    278,544 bytes, a 6-bit layer 409,616; window 2,112 bytes per head)."""
    assert head_bytes(4, 128, 128) == 8192 + 256 + 256 and head_bytes(6, 128, 128) == 12288 + 512
    assert head_bytes(2, 128, 128) == 4096 + 2 * 128 * 4 + 256 and head_bytes(16, 128, 128) == 32768
    w = torch.ones(32, 128)
    plan = StepPlan({l: (torch.tensor([[4, 6, 4, 4, 6, 4][l % 6]] * 32), w) for l in range(24)})
    pk = GGAPacked(plan, 32, 16, 128, 128, pw=True, m=8)
    assert pk.bytes_per_layer[0] == 278544 and pk.bytes_per_layer[1] == 409616
    assert pk.QSZ == 2112 and pk.QOFF == 409616 and pk.nbytes == 409616 + 32 * 2112 == 477200
    assert all(o % 16 == 0 for o in pk.tables[1][0])
    assert GGAPacked(plan, 32, 16, 128, 128, pw=False).nbytes == 409616


def _replay(c, name, stepper, loader, device):
    """Advance the packed master with ``stepper`` and compare every step with the reference emulation's record."""
    G = load_golden(name)
    pk, bits, w, blob = _setup(c, device)
    V = pk.views(blob)
    inp = {k: v.to(device) for k, v in gga_inputs(c).items()}
    idx = torch.tensor(c['idx'], dtype=torch.int32, device=device)
    ok = idx > 0
    hv, D, B = c['hv'], c['d'], c['B']
    return G, pk, V, inp, idx, ok


@pytest.mark.parametrize('name', list(GGA_CASES))
def test_oracle_step_matches_reference(name):
    c = GGA_CASES[name]
    G, pk, V, inp, idx, ok = _replay(c, name, None, None, 'cpu')
    oracle.gga_store(pk, V, idx[ok], inp['S0'], 0)
    hv, D, B = c['hv'], c['d'], c['B']
    piv = torch.tensor(c['widths']) == 16
    ki = 0
    for t in range(c['T']):
        out = torch.full((B, hv, D), 7.)
        oracle.gga_step(pk, V, idx, inp['q'][t], inp['k'][t], inp['v'][t], out, D ** -0.5,
                        (inp['a'][t], inp['b'][t], inp['A_log'], inp['dt_bias']), 0)
        want = torch.from_numpy(G['o'][t])
        assert torch.equal(out[~ok], torch.zeros_like(out[~ok]))
        assert ((out - want).norm() / want.norm()).item() < 1e-5, t
        if t in c['keep']:
            Sp = oracle.gga_load(pk, V, idx[ok], 0)
            Se = torch.from_numpy(G['O'][ki])
            flips = ((Sp - Se).abs() > 1e-3 * Se.abs().amax()).float().mean().item()
            assert flips < 2e-3, (t, flips)
            if c['pw']:
                P, Vw, n = pk.window(V, idx[ok])
                assert torch.equal(n, torch.from_numpy(G['n'][ki]).to(n.dtype)), t
                nonp = (~piv)[None, None, :, None]
                Pe, Ve = torch.from_numpy(G['P'][ki]), torch.from_numpy(G['V'][ki])
                z = torch.zeros(())
                P, Vw = torch.where(nonp, P, z), torch.where(nonp, Vw, z)      # pivot heads keep no window (garbage bytes)
                assert ((P - Pe * nonp).abs() > 1e-6 * P.abs().amax()).float().mean().item() < 1e-3, t
                assert torch.equal(Vw, Ve * nonp), t
            ki += 1


def test_pack_roundtrip_equals_fit():
    """load(store(x)) equals fit(x) for every width (reference: tests/test_gga_packed.py:36-50)."""
    c = dict(GGA_CASES['gga_step_pw'], widths=[2, 4, 6, 8], seed=61)
    pk, bits, w, blob = _setup(c)
    V = pk.views(blob)
    x = fit_input(64)[:, :4].contiguous()                           # [2, 4, dk, dv] canonical
    idx = torch.tensor([3, 1], dtype=torch.int32)
    oracle.gga_store(pk, V, idx, x.transpose(-1, -2), 0)
    assert torch.equal(oracle.gga_load(pk, V, idx, 0), oracle.stepquant_fit(x, bits, w))
    assert blob[idx.long(), :8].view(torch.int32).abs().sum() == 0


# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
def test_cuda_fit_matches_oracle():
    bits, w = gga_plan(5, 64, seed=3, widths=[2, 4, 6, 8, 16])
    x = fit_input(64)
    y = fit(x.to(DEV), bits.to(DEV), w.to(DEV)).cpu()
    want = oracle.stepquant_fit(x, bits, w)
    # the fit's column sums associate differently on the device: a refitted column factor can move by an fp16 ulp
    bad = ((y - want).abs() > 1e-3 * want.abs().amax()).float().mean().item()
    assert bad < 2e-3, bad
    assert torch.equal(y[:, 4], want[:, 4])                          # fp16 pivots: exact
    G = load_golden('gga_fit')
    ref = torch.from_numpy(G['y64'])
    assert ((y - ref).abs() > 1e-3 * ref.abs().amax()).float().mean().item() < 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize('name', list(GGA_CASES))
def test_cuda_step_matches_oracle_and_reference(name):
    """Every step from the same slot bytes through the CUDA kernels and the oracle: outputs, decoded state, window
    bytes; and the CUDA output against the reference emulation's record.  The master trajectory is the oracle's (the
    one the golden record was taken on), so the device starts each step from the master's bytes."""
    c = GGA_CASES[name]
    G, pk, Vh, inp, idx, ok = _replay(c, name, None, None, 'cpu')
    oracle.gga_store(pk, Vh, idx[ok], inp['S0'], 0)
    blob_d = Vh['blob'].clone().to(DEV)
    Vd = pk.views(blob_d)
    # the device packer on the same states gives the same decoded values up to refit flips
    blob_w = Vh['blob'].clone().to(DEV)
    Vw_ = pk.views(blob_w)
    pk.write(Vw_, idx[ok].to(DEV), inp['S0'].to(DEV), layer=0)
    a0, b0 = pk.stored(Vw_, idx[ok].to(DEV), 0).cpu(), oracle.gga_load(pk, Vh, idx[ok], 0)
    assert ((a0 - b0).abs() > 1e-3 * b0.abs().amax()).float().mean().item() < 2e-3
    hv, D, B = c['hv'], c['d'], c['B']
    piv = torch.tensor(c['widths']) == 16
    for t in range(c['T']):
        blob_d.copy_(Vh['blob'])                                    # both start every step from the master's bytes
        oh = torch.full((B, hv, D), 7.)
        od = torch.full((B, hv, D), 7., device=DEV)
        gate_h = (inp['a'][t], inp['b'][t], inp['A_log'], inp['dt_bias'])
        oracle.gga_step(pk, Vh, idx, inp['q'][t], inp['k'][t], inp['v'][t], oh, D ** -0.5, gate_h, 0)
        pk.step(Vd, idx.to(DEV), inp['q'][t].to(DEV), inp['k'][t].to(DEV), inp['v'][t].to(DEV), od, D ** -0.5,
                gate=tuple(x.to(DEV) for x in gate_h), layer=0)
        od = od.cpu()
        assert torch.equal(od[~ok], torch.zeros_like(od[~ok]))
        assert ((od - oh).norm() / oh.norm()).item() < 1e-5, t
        want = torch.from_numpy(G['o'][t])
        assert ((od - want).norm() / want.norm()).item() < 1e-5, t
        Sd, Sh = pk.stored(Vd, idx[ok].to(DEV), 0).cpu(), oracle.gga_load(pk, Vh, idx[ok], 0)
        flips = ((Sd - Sh).abs() > 1e-3 * Sh.abs().amax()).float().mean().item()
        assert flips < 2e-3, (t, flips)
        if c['pw']:
            Pd, Vwd, nd = pk.window(Vd, idx[ok].to(DEV))
            Ph, Vwh, nh = pk.window(Vh, idx[ok])
            assert torch.equal(nd.cpu(), nh)
            nonp = (~piv)[None, None, :, None]
            z = torch.zeros(())
            Pd, Vwd, Ph, Vwh = (torch.where(nonp, x_.cpu(), z) for x_ in (Pd, Vwd, Ph, Vwh))
            assert torch.equal(Vwd, Vwh), t
            assert ((Pd - Ph).abs() > 1e-6 * Ph.abs().amax()).float().mean().item() < 1e-3, t
    # bytes of slots that no row addressed are untouched
    untouched = [s for s in range(B + 2) if s not in [int(i) for i in idx if i > 0]]
    pk0, _, _, blob0 = _setup(c)
    assert torch.equal(blob_d.cpu()[untouched], blob0[untouched])


@pytest.mark.gpu
def test_cuda_graph_capture_gga():
    c = GGA_CASES['gga_step_pw']
    G, pk, Vh, inp, idx, ok = _replay(c, 'gga_step_pw', None, None, 'cpu')
    pk.prepare(DEV)
    blob = Vh['blob'].clone().to(DEV)
    V = pk.views(blob)
    idxd = idx.to(DEV)
    pk.write(V, idxd[ok.to(DEV)], inp['S0'].to(DEV), layer=0)
    snap = blob.clone()
    D, hv, B = c['d'], c['hv'], c['B']
    stat = [inp[k][0].clone().to(DEV) for k in ('q', 'k', 'v', 'a', 'b')]
    A_log, dtb = inp['A_log'].to(DEV), inp['dt_bias'].to(DEV)
    out = torch.empty(B, hv, D, device=DEV)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        pk.step(V, idxd, *stat[:3], out, D ** -0.5, gate=(stat[3], stat[4], A_log, dtb), layer=0)
    torch.cuda.current_stream().wait_stream(s)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        pk.step(V, idxd, *stat[:3], out, D ** -0.5, gate=(stat[3], stat[4], A_log, dtb), layer=0)
    blob.copy_(snap)
    eb = snap.clone()
    ev = pk.views(eb)
    oe = torch.empty_like(out)
    for t in range(c['T']):
        for dst, k in zip(stat, ('q', 'k', 'v', 'a', 'b')):
            dst.copy_(inp[k][t])
        gr.replay()
        pk.step(ev, idxd, *stat[:3], oe, D ** -0.5, gate=(stat[3], stat[4], A_log, dtb), layer=0)
        assert torch.equal(out, oe)
    assert torch.equal(blob, eb)


@pytest.mark.gpu
def test_full_batch_properties_gga_qwen_shapes():
    """Qwen3.5-4B head shapes (32 value heads, 16 key heads, 128 x 128), the 4 / 6-bit plan with the window, batch 64:
    determinism, padding rows, and a sample of slots against the oracle from their pre-step bytes across a window
    wrap (the queue fills at 8, merges start at 9)."""
    from statequant_b200.kernels.gga import StepPlan
    hv, hk, D, m, B = 32, 16, 128, 8, 64
    g0 = torch.Generator().manual_seed(11)
    plan = StepPlan({0: (torch.tensor([4, 6] * (hv // 2)), torch.rand(hv, D, generator=g0) + 0.5)}, 32, name='t')
    pk = GGAPacked(plan, hv, hk, D, D, pw=True, m=m)
    blob = pk.alloc(B + 1, DEV)
    V = pk.views(blob)
    idx = (torch.randperm(B, generator=g0) + 1).to(torch.int32)
    idx[::13] = 0
    idxd = idx.to(DEV)
    live = idxd[idxd > 0]
    pk.write(V, live, (torch.randn(int(live.numel()), hv, D, D, generator=g0) * 0.3).to(DEV), layer=0)
    blob2 = blob.clone()
    V2 = pk.views(blob2)
    sample = [int(s) for s in idx[1:4] if s > 0]
    rows = [int((idx == s).nonzero()[0]) for s in sample]
    A_log, dtb = torch.randn(hv, generator=g0) * 0.3, torch.randn(hv, generator=g0)
    for t in range(m + 2):
        f = lambda *s: torch.randn(*s, generator=g0)                                     # noqa: E731
        q, k, v = f(B, hk, D).bfloat16(), f(B, hk, D).bfloat16(), f(B, hv, D).bfloat16()
        a, b = (f(B, hv) + 2.0).bfloat16(), f(B, hv).bfloat16()
        out = torch.empty(B, hv, D, dtype=torch.bfloat16, device=DEV)
        out2 = torch.empty_like(out)
        pre = blob[torch.tensor(sample, device=DEV)].cpu()
        gate = tuple(x.to(DEV) for x in (a, b, A_log, dtb))
        args = [x.to(DEV) for x in (q, k, v)]
        pk.step(V, idxd, *args, out, D ** -0.5, gate=gate, layer=0)
        pk.step(V2, idxd, *args, out2, D ** -0.5, gate=gate, layer=0)
        assert torch.equal(out, out2) and torch.equal(blob, blob2), t
        assert torch.equal(out[idxd <= 0], torch.zeros_like(out[idxd <= 0]))
        hb = torch.zeros(B + 1, blob.shape[1], dtype=torch.uint8)
        hb[torch.tensor(sample)] = pre
        Vh = pk.views(hb)
        oh = torch.empty(len(rows), hv, D, dtype=torch.bfloat16)
        oracle.gga_step(pk, Vh, idx[rows].contiguous(), q[rows].contiguous(), k[rows].contiguous(), v[rows].contiguous(),
                        oh, D ** -0.5, (a[rows].contiguous(), b[rows].contiguous(), A_log, dtb), 0)
        assert torch.allclose(out[rows].cpu().float(), oh.float(), rtol=1e-2, atol=2e-3), t
        sl = torch.tensor(sample, dtype=torch.int32)
        Sd = pk.stored(V, sl.to(DEV), 0).cpu()
        Sh = oracle.gga_load(pk, Vh, sl, 0)
        flips = ((Sd - Sh).abs() > 1e-3 * Sh.abs().amax()).float().mean().item()
        assert flips < 2e-3, (t, flips)
        assert torch.equal(blob.cpu()[sl.long(), :8], hb[sl.long(), :8])               # window counters


@pytest.mark.gpu
@pytest.mark.parametrize('pw', [True, False])
def test_mixed_widths_at_128_split_between_the_two_step_kernels(pw):
    """A 128 x 128 layer that mixes the widths: 4 / 6 / 8-bit heads go to the register-tile kernel, the 2-bit head and the
    fp16 pivot to the tile kernel (the layout carries no all-packed hint here), every step from the oracle's bytes,
    across a window wrap (m = 4), with padding rows; then the same layer with the generic path forced (tile kernel for
    every head) must give the device's own bytes again up to refit flips."""
    from statequant_b200 import _cabi
    hv, hk, D, m, B = 6, 3, 128, 4, 3
    g0 = torch.Generator().manual_seed(77)
    widths = torch.tensor([8, 16, 2, 4, 6, 8])
    plan = StepPlan({0: (widths, torch.rand(hv, D, generator=g0) + 0.5)}, 32, name='mixed')
    pk = GGAPacked(plan, hv, hk, D, D, pw=pw, m=m)
    assert pk._struct(pk.views(torch.zeros(1, pk.nbytes, dtype=torch.uint8)), 0).flags == 0
    idx = torch.tensor([2, 0, 1], dtype=torch.int32)
    ok = idx > 0
    hb = torch.zeros(B + 1, pk.nbytes, dtype=torch.uint8)
    Vh = pk.views(hb)
    oracle.gga_store(pk, Vh, idx[ok], torch.randn(int(ok.sum()), hv, D, D, generator=g0) * 0.3, 0)
    db = hb.clone().to(DEV)
    Vd = pk.views(db)
    A_log, dtb = torch.randn(hv, generator=g0) * 0.3, torch.randn(hv, generator=g0)
    packed = (widths != 16) & (widths != 2)
    for t in range(2 * m + 1):
        f = lambda *s: torch.randn(*s, generator=g0)                                     # noqa: E731
        q, k, v = f(B, hk, D), f(B, hk, D), f(B, hv, D)
        a, b = f(B, hv) + 2.0, f(B, hv)
        db.copy_(hb)                                             # both start from the master's bytes
        oh = torch.full((B, hv, D), 7.)
        od = torch.full((B, hv, D), 7., device=DEV)
        oracle.gga_step(pk, Vh, idx, q, k, v, oh, D ** -0.5, (a, b, A_log, dtb), 0)
        gate = tuple(x.to(DEV) for x in (a, b, A_log, dtb))
        pk.step(Vd, idx.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), od, D ** -0.5, gate=gate, layer=0)
        od = od.cpu()
        assert torch.equal(od[~ok], torch.zeros_like(od[~ok]))
        assert ((od - oh).norm() / oh.norm()).item() < 1e-5, t
        Sd, Sh = pk.stored(Vd, idx[ok].to(DEV), 0).cpu(), oracle.gga_load(pk, Vh, idx[ok], 0)
        flips = ((Sd - Sh).abs() > 1e-3 * Sh.abs().amax()).float().mean().item()
        assert flips < 2e-3, (t, flips)
        if pw:
            Pd, Vwd, nd = pk.window(Vd, idx[ok].to(DEV))
            Ph, Vwh, nh = pk.window(Vh, idx[ok])
            assert torch.equal(nd.cpu(), nh) and torch.equal(Vwd.cpu(), Vwh), t
            assert ((Pd.cpu() - Ph).abs() > 1e-6 * Ph.abs().amax()).float().mean().item() < 1e-3, t
        assert torch.equal(db.cpu()[0], hb[0])                   # the padding slot is untouched
    # the tile kernel alone on the last step's inputs gives the same outputs
    db.copy_(hb)
    o1 = torch.empty(B, hv, D, device=DEV)
    pk.step(Vd, idx.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), o1, D ** -0.5, gate=gate, layer=0)
    db.copy_(hb)
    o2 = torch.empty(B, hv, D, device=DEV)
    _cabi.set_option('kernel_path', 1)
    try:
        pk.step(Vd, idx.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), o2, D ** -0.5, gate=gate, layer=0)
    finally:
        _cabi.set_option('kernel_path', 0)
    assert ((o1 - o2).norm() / o2.norm()).item() < 1e-5
    assert torch.equal(o1[:, ~packed], o2[:, ~packed])           # heads the tile kernel serves either way: identical


@pytest.mark.gpu
@pytest.mark.parametrize('scale', [1e16, 3e13])
def test_register_tile_kernel_outside_the_fast_quotient_range(scale):
    """Values for which the fit's three-FMA quotients are not proved exact: the register-tile kernel must take its IEEE
    path for the head.  A value vector of 1e16 drives a head's row sums past 1e14; one of 3e13 in a single column cuts a column factor at
    fp16's maximum (quotients pass the code range; the row sums stay below 1e14).  No window, so the write lands in the state at once."""
    hv, hk, D, B = 2, 1, 128, 2
    g0 = torch.Generator().manual_seed(5)
    plan = StepPlan({0: (torch.tensor([4, 8]), torch.rand(hv, D, generator=g0) + 0.5)}, 32, name='range')
    pk = GGAPacked(plan, hv, hk, D, D, pw=False, m=8)
    idx = torch.tensor([1, 2], dtype=torch.int32)
    hb = torch.zeros(B + 1, pk.nbytes, dtype=torch.uint8)
    Vh = pk.views(hb)
    oracle.gga_store(pk, Vh, idx, torch.randn(B, hv, D, D, generator=g0) * 0.3, 0)
    db = hb.clone().to(DEV)
    Vd = pk.views(db)
    A_log, dtb = torch.randn(hv, generator=g0) * 0.3, torch.randn(hv, generator=g0)
    for t in range(3):
        f = lambda *s: torch.randn(*s, generator=g0)                                     # noqa: E731
        q, k, v = f(B, hk, D), f(B, hk, D), f(B, hv, D)
        v[0, 1] *= scale                                          # row 0, head 1: out of range; the others stay in it
        if scale < 1e15:
            v[0, 1, 1:] = 0.                                      # one huge column only
        a, b = f(B, hv) + 2.0, f(B, hv)
        db.copy_(hb)
        oh, od = torch.empty(B, hv, D), torch.empty(B, hv, D, device=DEV)
        oracle.gga_step(pk, Vh, idx, q, k, v, oh, D ** -0.5, (a, b, A_log, dtb), 0)
        pk.step(Vd, idx.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), od, D ** -0.5,
                gate=tuple(x.to(DEV) for x in (a, b, A_log, dtb)), layer=0)
        assert torch.isfinite(od).all()
        assert ((od.cpu() - oh).norm() / oh.norm()).item() < 1e-5, t
        Sd, Sh = pk.stored(Vd, idx.to(DEV), 0).cpu(), oracle.gga_load(pk, Vh, idx, 0)
        for h in range(hv):
            for r in range(B):
                ref = Sh[r, h]
                flips = ((Sd[r, h] - ref).abs() > 1e-3 * ref.abs().amax()).float().mean().item()
                assert flips < 2e-3, (t, r, h, flips)


@pytest.mark.gpu
def test_register_tile_kernel_bounded_wait_runs_out_and_is_reported():
    """The register-tile kernel's wait for its two bulk copies is bounded like the step kernels': with the barrier told
    to expect more bytes than are copied (test switch) and a short limit, every CTA gives up together, the health word
    counts them, the output rows are zero and the slots are untouched; afterwards the library works as before."""
    from statequant_b200 import _cabi
    hv, hk, D, B = 4, 2, 128, 2
    g0 = torch.Generator().manual_seed(9)
    plan = StepPlan({0: (torch.tensor([4, 6, 8, 4]), torch.rand(hv, D, generator=g0) + 0.5)}, 32, name='wait')
    pk = GGAPacked(plan, hv, hk, D, D, pw=True, m=4)
    blob = pk.alloc(B + 1, DEV)
    V = pk.views(blob)
    idx = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
    pk.write(V, idx, (torch.randn(B, hv, D, D, generator=g0) * 0.3).to(DEV), layer=0)
    f = lambda *s: torch.randn(*s, generator=g0).to(DEV)                                 # noqa: E731
    q, k, v, a, b = f(B, hk, D), f(B, hk, D), f(B, hv, D), f(B, hv) + 2.0, f(B, hv)
    gate = (a, b, f(hv) * 0.3, f(hv))
    out = torch.full((B, hv, D), 7., device=DEV)
    pk.step(V, idx, q, k, v, out, D ** -0.5, gate=gate, layer=0)                         # a healthy step first
    torch.cuda.synchronize()
    base = _cabi.device_status()
    before = blob.clone()
    _cabi.set_option('wait_limit_us', 2000)
    _cabi.set_option('test_extra_tx', 64)
    try:
        out.fill_(7.)
        pk.step(V, idx, q, k, v, out, D ** -0.5, gate=gate, layer=0)
        torch.cuda.synchronize()
        assert _cabi.device_status() - base == B * hv                                    # one count per CTA
        assert torch.equal(out, torch.zeros_like(out))
        assert torch.equal(blob[:, 16:], before[:, 16:])                                 # heads and windows untouched
    finally:
        _cabi.set_option('test_extra_tx', 0)
        _cabi.set_option('wait_limit_us', 1000000)
    blob.copy_(before)
    o2 = torch.empty_like(out)
    pk.step(V, idx, q, k, v, o2, D ** -0.5, gate=gate, layer=0)
    torch.cuda.synchronize()
    assert _cabi.device_status() - base == B * hv and torch.isfinite(o2).all() and o2.abs().sum() > 0
