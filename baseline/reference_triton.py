"""The reference's own Triton path on this GPU, next to the sm_100a kernels: timing with the reference's protocol and a
byte comparison of the stored state.

    python baseline/reference_triton.py [--batch 256] [--layers 8] [--out FILE.json]

Needs the reference package installed under baseline/_ref (baseline/install_reference.sh) and Triton able to JIT for
the GPU; prints one JSON document (and writes it to --out).  If the reference or Triton is unusable, the document says
why and the exit code is 0.

Timing: per layer per decode step, a CUDA graph of m = 8 consecutive steps (exactly one fold) divided by 8, minimum
over 20 repeats, CUDA events: the protocol of the reference's benchmarks/decode_state.py:41-66.  The reference times
ONE layer, whose state (84 to 156 MB at batch 256) is largely L2-resident on this GPU; the same figure is therefore
also taken over `--layers` layers stepped in turn (working set far above L2), for both implementations.

Bytes: from identical seeded inputs and an identical initial blob (written by the reference's own `write`), both step
2 m + 1 tokens; the blobs are compared field by field.  For the GGA state the comparison is of `write` (the STEP fit and
the packer): the reference's packer exists only as a Triton kernel, so this is what pins the order of code bytes.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, 'baseline', '_ref')


def time_graph(fn, steps=8, repeats=20, inner=5):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2 * steps):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(steps):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    best = float('inf')
    for _ in range(repeats):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(inner):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) * 1e3 / (inner * steps))
    return best


def gdn_inputs(B, hk, hv, d, gen, dev):
    f = lambda *s: torch.randn(*s, generator=gen)                                        # noqa: E731
    return [t.to(dev) for t in (f(B, hk, d).bfloat16(), f(B, hk, d).bfloat16(), f(B, hv, d).bfloat16(),
                                (f(B, hv) + 2.0).bfloat16(), f(B, hv).bfloat16())]


def field_mismatch(lay, a, b, slots):
    """{field: (differing elements, elements)} of two blobs over the live slots; 4-bit codes are counted per code."""
    va, vb = lay.views(a), lay.views(b)
    out = {}
    for name in va:
        x, y = va[name][slots].contiguous(), vb[name][slots].contiguous()
        if name == 'S' and getattr(lay, 'bits', 8) == 4:
            n = int(((x & 15) != (y & 15)).sum() + ((x >> 4) != (y >> 4)).sum())
            out[name] = (n, x.numel() * 2)
            continue
        xi, yi = x.view(torch.uint8), y.view(torch.uint8)
        w = x.element_size()
        out[name] = (int((xi.view(-1, w) != yi.view(-1, w)).any(dim=1).sum()), x.numel())
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--batch', type=int, default=256)
    ap.add_argument('--layers', type=int, default=8)
    ap.add_argument('--out', default=None)
    args = ap.parse_args()
    doc = {'what': 'the reference Triton kernels and the sm_100a kernels on the same GPU', 'batch': args.batch}

    def finish():
        s = json.dumps(doc, indent=1)
        print(s)
        if args.out:
            with open(args.out, 'w') as f:
                f.write(s + '\n')

    if not os.path.isdir(os.path.join(REF, 'statequant')):
        doc['unavailable'] = 'baseline/_ref holds no reference install (run baseline/install_reference.sh)'
        return finish()
    if not torch.cuda.is_available():
        doc['unavailable'] = 'no CUDA device'
        return finish()
    sys.path.insert(0, REF)
    sys.path.insert(0, ROOT)
    import statequant as rsq
    from statequant import kernels as RK
    import statequant_b200 as sq
    from statequant_b200 import kernels as K
    dev = 'cuda'
    doc['gpu'] = torch.cuda.get_device_name(0)
    B, HV, HK, D, M = args.batch, 32, 16, 128, 8
    gen = torch.Generator().manual_seed(777)

    # ---------------------------------------------------------------- GDN: bytes, then timing, per preset
    doc['gdn'] = {}
    for preset, fmt in (('int8k', (8, 'k', 32)), ('pace4', (4, 'k', 64)), ('int4v', (4, 'v', 32))):
        rec = doc['gdn'][preset] = {}
        try:
            rlay = RK.SlotLayout(rsq.Quantizer(*fmt), HV, HK, D, D, m=M, buffer_bits=8)
            olay = K.SlotLayout(sq.Quantizer(*fmt), HV, HK, D, D, m=M, buffer_bits=8)
            assert rlay.nbytes == olay.nbytes
            nb = 9
            S0 = (torch.randn(nb - 1, HV, D, D, generator=gen) * 0.3).to(dev)
            blob_r = torch.zeros(nb, rlay.nbytes, dtype=torch.uint8, device=dev)
            slots = torch.arange(1, nb, device=dev)
            rlay.write(rlay.views(blob_r), slots, S0)                 # the reference's own packer
            blob_o = blob_r.clone()
            idx = torch.arange(1, nb, dtype=torch.int32, device=dev)
            A_log, dtb = (torch.randn(HV, generator=gen) * 0.3).to(dev), torch.randn(HV, generator=gen).to(dev)
            worst = 0.
            for t in range(2 * M + 1):
                q, k, v, a, b = gdn_inputs(nb - 1, HK, HV, D, gen, dev)
                o_r = torch.empty(nb - 1, HV, D, dtype=torch.bfloat16, device=dev)
                o_o = torch.empty_like(o_r)
                rlay.step(rlay.views(blob_r), idx, q, k, v, o_r, D ** -0.5, gate=(a, b, A_log, dtb))
                olay.step(olay.views(blob_o), idx, q, k, v, o_o, D ** -0.5, gate=(a, b, A_log, dtb))
                worst = max(worst, float((o_r.float() - o_o.float()).abs().max() / o_r.float().abs().max()))
            torch.cuda.synchronize()
            rec['bytes_after_17_steps'] = {k_: list(v_) for k_, v_ in field_mismatch(olay, blob_o, blob_r, slots).items()}
            rec['max_rel_output_diff_bf16'] = worst
        except Exception as e:                                          # Triton may not JIT for this GPU
            rec['unavailable'] = f'{type(e).__name__}: {str(e)[:300]}'
            continue
        # timing: one layer (the reference's protocol) and args.layers layers in turn
        for which, lay in (('reference_triton', rlay), ('sm100a', olay)):
            for L in (1, args.layers):
                blobs = [lay.alloc(B + 1, dev) for _ in range(L)]
                views = [lay.views(x) for x in blobs]
                ins = [gdn_inputs(B, HK, HV, D, gen, dev) for _ in range(L)]
                outs = [torch.empty(B, HV, D, dtype=torch.bfloat16, device=dev) for _ in range(L)]
                idxb = (torch.randperm(B, generator=gen) + 1).to(torch.int32).to(dev)

                def step():
                    for l in range(L):
                        q, k, v, a, b = ins[l]
                        lay.step(views[l], idxb, q, k, v, outs[l], D ** -0.5, gate=(a, b, A_log, dtb))
                for _ in range(64):
                    step()
                rec[f'{which}_us_per_layer_step_{L}_layers'] = time_graph(step) / L
                del blobs, views
                torch.cuda.empty_cache()

    # ---------------------------------------------------------------- Mamba2 and KDA: timing and bytes
    try:
        H, GR, DS, HD = 128, 8, 128, 64
        fmt = (8, 'k', 32)
        rl = RK.Mamba2SlotLayout(rsq.Quantizer(*fmt), H, GR, DS, HD, m=M, buffer_bits=8)
        ol = K.Mamba2SlotLayout(sq.Quantizer(*fmt), H, GR, DS, HD, m=M, buffer_bits=8)
        A = (-torch.exp(torch.rand(H, generator=gen) * 2.77)).to(dev)
        Dp, dtb2 = torch.randn(H, generator=gen).to(dev), (torch.rand(H, generator=gen) * 2 - 4).to(dev)
        rec = doc['mamba2_int8k'] = {}
        f = lambda *s: torch.randn(*s, generator=gen)                                    # noqa: E731
        nb = 5
        br = torch.zeros(nb, rl.nbytes, dtype=torch.uint8, device=dev)
        sl = torch.arange(1, nb, device=dev)
        rl.write(rl.views(br), sl, (f(nb - 1, H, HD, DS) * 0.3).to(dev))
        bo = br.clone()
        idx = torch.arange(1, nb, dtype=torch.int32, device=dev)
        for t in range(2 * M + 1):
            x, dt, Bm, Cm = (f(nb - 1, H, HD).bfloat16().to(dev), f(nb - 1, H).bfloat16().to(dev),
                             f(nb - 1, GR, DS).bfloat16().to(dev), f(nb - 1, GR, DS).bfloat16().to(dev))
            o1 = torch.empty(nb - 1, H, HD, dtype=torch.bfloat16, device=dev)
            o2 = torch.empty_like(o1)
            rl.step(rl.views(br), idx, x, dt, Bm, Cm, o1, A, D=Dp, dt_bias=dtb2)
            ol.step(ol.views(bo), idx, x, dt, Bm, Cm, o2, A, D=Dp, dt_bias=dtb2)
        torch.cuda.synchronize()
        rec['bytes_after_17_steps'] = {k_: list(v_) for k_, v_ in field_mismatch(ol, bo, br, sl).items()}
        for which, lay in (('reference_triton', rl), ('sm100a', ol)):
            L = 4
            blobs = [lay.alloc(B + 1, dev) for _ in range(L)]
            views = [lay.views(x_) for x_ in blobs]
            ins = [(f(B, H, HD).bfloat16().to(dev), f(B, H).bfloat16().to(dev), f(B, GR, DS).bfloat16().to(dev),
                    f(B, GR, DS).bfloat16().to(dev)) for _ in range(L)]
            outs = [torch.empty(B, H, HD, dtype=torch.bfloat16, device=dev) for _ in range(L)]
            idxb = (torch.randperm(B, generator=gen) + 1).to(torch.int32).to(dev)

            def step():
                for l in range(L):
                    x, dt, Bm, Cm = ins[l]
                    lay.step(views[l], idxb, x, dt, Bm, Cm, outs[l], A, D=Dp, dt_bias=dtb2)
            for _ in range(32):
                step()
            rec[f'{which}_us_per_layer_step_{L}_layers'] = time_graph(step) / L
            del blobs, views
            torch.cuda.empty_cache()
    except Exception as e:
        doc['mamba2_int8k'] = {'unavailable': f'{type(e).__name__}: {str(e)[:300]}'}

    try:
        Hk = 32
        fmt = (4, 'k', 64)
        rl = RK.KDASlotLayout(rsq.Quantizer(*fmt), Hk, D, D, m=M, buffer_bits=8)
        ol = K.KDASlotLayout(sq.Quantizer(*fmt), Hk, D, D, m=M, buffer_bits=8)
        rec = doc['kda_pace4'] = {}
        f = lambda *s: torch.randn(*s, generator=gen)                                    # noqa: E731

        def kin(n):
            q, k = f(n, Hk, D), f(n, Hk, D)
            return [t.to(dev) for t in ((q / q.norm(dim=-1, keepdim=True)).bfloat16(), (k / k.norm(dim=-1, keepdim=True)).bfloat16(),
                                        f(n, Hk, D).bfloat16(), torch.nn.functional.logsigmoid(f(n, Hk, D) + 3.0), torch.sigmoid(f(n, Hk)))]
        nb = 5
        br = torch.zeros(nb, rl.nbytes, dtype=torch.uint8, device=dev)
        sl = torch.arange(1, nb, device=dev)
        rl.write(rl.views(br), sl, (f(nb - 1, Hk, D, D) * 0.3).to(dev))
        bo = br.clone()
        idx = torch.arange(1, nb, dtype=torch.int32, device=dev)
        for t in range(2 * M + 1):
            q, k, v, g, be = kin(nb - 1)
            o1 = torch.empty(nb - 1, Hk, D, dtype=torch.bfloat16, device=dev)
            o2 = torch.empty_like(o1)
            rl.step(rl.views(br), idx, q, k, v, g, be, o1, D ** -0.5)
            ol.step(ol.views(bo), idx, q, k, v, g, be, o2, D ** -0.5)
        torch.cuda.synchronize()
        rec['bytes_after_17_steps'] = {k_: list(v_) for k_, v_ in field_mismatch(ol, bo, br, sl).items()}
        for which, lay in (('reference_triton', rl), ('sm100a', ol)):
            L = 8
            blobs = [lay.alloc(B + 1, dev) for _ in range(L)]
            views = [lay.views(x_) for x_ in blobs]
            ins = [kin(B) for _ in range(L)]
            outs = [torch.empty(B, Hk, D, dtype=torch.bfloat16, device=dev) for _ in range(L)]
            idxb = (torch.randperm(B, generator=gen) + 1).to(torch.int32).to(dev)

            def step():
                for l in range(L):
                    q, k, v, g, be = ins[l]
                    lay.step(views[l], idxb, q, k, v, g, be, outs[l], D ** -0.5)
            for _ in range(32):
                step()
            rec[f'{which}_us_per_layer_step_{L}_layers'] = time_graph(step) / L
            del blobs, views
            torch.cuda.empty_cache()
    except Exception as e:
        doc['kda_pace4'] = {'unavailable': f'{type(e).__name__}: {str(e)[:300]}'}

    # ---------------------------------------------------------------- GGA: the packer's bytes, and the step's time
    try:
        from statequant.integrations.vllm_gga import GGAPacked as RGGA
        import types
        widths = [4, 6, 4, 4, 6, 4]
        nl = 6
        plan = {L_: (torch.full((HV,), widths[L_ % 6]), torch.rand(HV, D, generator=gen) + 0.5) for L_ in range(nl)}
        rg = RGGA(types.SimpleNamespace(plan=plan, group=32, name='probe'), HV, HK, D, D, pw=True, m=8)
        from statequant_b200.kernels.gga import StepPlan
        og = K.GGAPacked(StepPlan(plan, 32), HV, HK, D, D, pw=True, m=8)
        rec = doc['gga'] = {'nbytes': [rg.nbytes, og.nbytes]}
        nb = 5
        S0 = (torch.randn(nb - 1, HV, D, D, generator=gen) * 0.3).to(dev)
        sl = torch.arange(1, nb, device=dev)
        for layer in (0, 1):
            br = torch.zeros(nb, rg.nbytes, dtype=torch.uint8, device=dev)
            bo = torch.zeros(nb, og.nbytes, dtype=torch.uint8, device=dev)
            rg.write(rg.views(br), sl, S0, layer=layer)
            og.write(og.views(bo), sl, S0, layer=layer)
            torch.cuda.synchronize()
            n = min(rg.nbytes, og.nbytes)
            rec[f'write_layer{layer}_{widths[layer]}bit_differing_bytes'] = [int((br[1:, :n] != bo[1:, :n]).sum()), int(br[1:, :n].numel())]
            # a few decode tokens from the reference's bytes through both (past the window's fill: 10 tokens)
            bo.copy_(br)
            idx = torch.arange(1, nb, dtype=torch.int32, device=dev)
            A_log, dtb = (torch.randn(HV, generator=gen) * 0.3).to(dev), torch.randn(HV, generator=gen).to(dev)
            worst = 0.
            for t in range(10):
                q, k, v, a, b = gdn_inputs(nb - 1, HK, HV, D, gen, dev)
                o1 = torch.empty(nb - 1, HV, D, dtype=torch.bfloat16, device=dev)
                o2 = torch.empty_like(o1)
                rg.step(rg.views(br), idx, q, k, v, o1, D ** -0.5, gate=(a, b, A_log, dtb), layer=layer)
                og.step(og.views(bo), idx, q, k, v, o2, D ** -0.5, gate=(a, b, A_log, dtb), layer=layer)
                worst = max(worst, float((o1.float() - o2.float()).abs().max() / o1.float().abs().max()))
            torch.cuda.synchronize()
            rec[f'step_layer{layer}_differing_bytes_after_10_tokens'] = [int((br[1:, :n] != bo[1:, :n]).sum()), int(br[1:, :n].numel())]
            rec[f'step_layer{layer}_max_rel_output_diff_bf16'] = worst
    except Exception as e:
        doc['gga'] = {'unavailable': f'{type(e).__name__}: {str(e)[:400]}'}
    finish()


if __name__ == '__main__':
    main()
