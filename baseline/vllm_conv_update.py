"""vLLM's own `causal_conv1d_update` (Triton) on this GPU next to the sm_100a kernel: timing and a byte comparison.

    python baseline/vllm_conv_update.py [--batch 256] [--layers 24] [--out FILE.json]

The op is the one the reference's vLLM forward calls right before the packed step
(src/statequant/integrations/vllm_plugin.py:379-381 in the reference).  Shapes: the GDN layer of the benchmark
(2 x 16 x 128 + 32 x 128 = 8192 channels, width 4, bf16, SiLU), the cache as vLLM lays it out ([lines, 3, dim]).
Timing: one cache per layer (24 x 12.6 MB, above L2), a CUDA graph of one call per layer, CUDA events, microseconds per
call.  Bytes: both implementations advance identical caches by three tokens; the caches must be equal, the outputs are
compared as bf16 bit patterns.  If vLLM or Triton is unusable the document says why and the exit code is 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def time_calls(fn, layers, reps=10):
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (reps * layers)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--batch', type=int, default=256)
    ap.add_argument('--layers', type=int, default=24)
    ap.add_argument('--out', default=None)
    args = ap.parse_args()
    doc = {'batch': args.batch, 'layers': args.layers}
    try:
        from vllm.model_executor.layers.mamba.ops.causal_conv1d import causal_conv1d_update as vllm_update
    except Exception as err:
        doc['unavailable'] = f'vLLM op not importable: {err!r}'
        print(json.dumps(doc))
        return
    from statequant_b200.kernels import causal_conv1d_update
    dev = 'cuda:0'
    gen = torch.Generator().manual_seed(5)
    dim, width, B = 8192, 4, args.batch
    w = (torch.randn(dim, width, generator=gen) * 0.5).to(torch.bfloat16).to(dev)
    bias = (torch.randn(dim, generator=gen) * 0.1).to(torch.bfloat16).to(dev)
    idx = (torch.randperm(B, generator=gen) + 1).to(torch.int32).to(dev)
    caches = [torch.randn(B + 1, width - 1, dim, generator=gen).to(torch.bfloat16).to(dev) for _ in range(args.layers)]
    xs = [torch.randn(B, dim, generator=gen).to(torch.bfloat16).to(dev) for _ in range(args.layers)]

    # bytes: three tokens through one cache, both ways
    mine_c, ref_c = caches[0].clone(), caches[0].clone()
    mine_x, ref_x = xs[0].clone(), xs[0].clone()
    try:
        diff = []
        for _ in range(3):
            ro = vllm_update(ref_x, ref_c.transpose(1, 2), w, bias, 'silu', conv_state_indices=idx)
            mo = causal_conv1d_update(mine_x, mine_c.transpose(1, 2), w, bias, 'silu', idx)
            d = (mo.view(torch.int16).int() - ro.view(torch.int16).int()).abs()
            diff.append({'outputs_differing': int((d > 0).sum()), 'of': d.numel(), 'max_units_in_last_place': int(d.max()),
                         'cache_bytes_differing': int((mine_c.view(torch.uint8) != ref_c.view(torch.uint8)).sum())})
            mine_x.copy_(ro)
            ref_x.copy_(ro)
        doc['bytes'] = diff
        doc['vllm_us_per_call'] = time_calls(lambda: [vllm_update(x, c.transpose(1, 2), w, bias, 'silu', conv_state_indices=idx)
                                                      for x, c in zip(xs, caches)], args.layers)
    except Exception as err:
        doc['unavailable'] = f'vLLM op did not run: {err!r}'
    doc['this_package_us_per_call'] = time_calls(lambda: [causal_conv1d_update(x, c.transpose(1, 2), w, bias, 'silu', idx)
                                                          for x, c in zip(xs, caches)], args.layers)
    doc['algorithmic_bytes_per_call'] = B * dim * 2 * (2 * (width - 1) + 2)
    print(json.dumps(doc))
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        json.dump(doc, open(args.out, 'w'), indent=1)


if __name__ == '__main__':
    main()
