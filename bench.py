#!/usr/bin/env python
"""Benchmark of the fused packed-state decode step.

Workload (the configuration the metric is quoted on): the 24-layer Gated DeltaNet decode stack at Qwen3.5-4B
shapes -- 32 value heads, 16 key heads, d_k = d_v = 128, buffer length 8 with an int8 buffer -- batch 256 slots per
GPU, bf16 activations with in-kernel gating, the state stored int8 (preset int8k: key-axis groups of 32); int4v and
pace4 are timed as secondary variants.  Every slot is pre-warmed by random steps drawn from the same distributions.
A "step" is one decode token for the whole batch through all 24 layers (24 launches); the metric counts
layer-steps (one layer advancing one token for the batch) per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints one JSON line (rank 0).  With N > 1 it is launched under torchrun, one process per GPU: slots are
independent, so each rank owns its own 256 slots and there is no data-path collective (weak scaling).
``--impl reference`` times the CPU restatement of the reference's torch path (the oracle) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, 'tests')):
    if p not in sys.path:
        sys.path.insert(0, p)

import math  # noqa: E402

import torch  # noqa: E402

HV, HK, DK, DV, M = 32, 16, 128, 128, 8
LAYERS = 24          # overridden by --layers (profiling runs use fewer)
PRESETS = {'int8k': (8, 'k', 32), 'int4v': (4, 'v', 32), 'pace4': (4, 'k', 64)}
EXTRA_PRESETS = {'int8v': (8, 'v', 32)}             # not in the default run: --preset int8v --no-variants
METRIC = 'decode layer-steps/s (24-layer GDN stack, batch 256 slots per GPU)'
UNIT = 'layer-steps/s'


def algorithmic_bytes(lay):
    """Bytes one (slot, layer, step) must move, averaged over a fold period of m steps: the stored state read every
    step and rewritten once per m, the live half of the buffer, the appended entry, counters, bf16 inputs and
    output."""
    b = lay.breakdown()
    m = lay.m
    state = (b['S'] + b.get('SC', 0)) * (1 + 1 / m)
    buf = b['KB'] + b['UB'] + b.get('KBS', 0) + b.get('UBS', 0) + b['GB']
    io = 2 * (2 * lay.HK * lay.DK + lay.HV * lay.DV + 2 * lay.HV) + 2 * lay.HV * lay.DV
    total = state + buf * (m - 1) / (2 * m) + buf / m + 2 * (b['GCUR'] + b['NPTR']) + io
    return total, state


def make_inputs(batch, gen, device, pinned=False):
    """One layer's activations, bf16: q, k l2-normalised N(0,1) per key head, v ~ N(0,1), gate inputs a, b."""
    f = lambda *s: torch.randn(*s, generator=gen)                                        # noqa: E731
    q, k = f(batch, HK, DK), f(batch, HK, DK)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    t = [q.bfloat16(), k.bfloat16(), f(batch, HV, DV).bfloat16(), (f(batch, HV) + 2.0).bfloat16(), f(batch, HV).bfloat16()]
    if pinned:
        return [x.pin_memory() for x in t]
    return [x.to(device) for x in t]


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while the timed region runs."""
    Q = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
         'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
         'clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits',
                                          '-lms', '200', '-i', str(index)], stdout=subprocess.PIPE, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(',')]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.25)
        self.proc.terminate()
        rows = [r for ts, r in self.rows if t0 <= ts <= t1 + 0.2 and len(r) >= 7] or [r for _, r in self.rows if len(r) >= 7]
        if not rows:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['no samples']}
        sm = sorted(float(r[0]) for r in rows)
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith('active') for r in rows)]
        return {'sm_mhz': sm[len(sm) // 2], 'sm_max_mhz': float(rows[0][1]), 'reasons': reasons,
                'samples': len(rows), 'power_w_max': max(float(r[2]) for r in rows)}


def measured_peak_gbs():
    try:
        return float(json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json')))['hbm_gbs']), 'measured'
    except Exception:
        return 6650.0, 'fallback'


class Stack:
    """The 24-layer stack of one preset on one GPU: blobs, resident inputs, a CUDA graph of one decode step."""

    def __init__(self, preset, batch, device, seed):
        import statequant_b200 as sq
        from statequant_b200.kernels import SlotLayout
        self.lay = SlotLayout(sq.Quantizer(*{**PRESETS, **EXTRA_PRESETS}[preset]), HV, HK, DK, DV, m=M, buffer_bits=8)
        self.batch, self.device = batch, device
        gen = torch.Generator().manual_seed(seed)
        self.blobs = [self.lay.alloc(batch + 1, device) for _ in range(LAYERS)]
        self.views = [self.lay.views(b) for b in self.blobs]
        self.idx = (torch.randperm(batch, generator=gen) + 1).to(torch.int32).to(device)     # slot 0 is padding
        self.inputs = [make_inputs(batch, gen, device) for _ in range(LAYERS)]
        self.A_log = (torch.randn(HV, generator=gen) * 0.3).to(device)
        self.dt_bias = torch.randn(HV, generator=gen).to(device)
        self.outs = [torch.empty(batch, HV, DV, dtype=torch.bfloat16, device=device) for _ in range(LAYERS)]
        self.graph = None
        self.launches_per_step = None

    def bytes_per_slot(self):
        return algorithmic_bytes(self.lay)

    def step(self):
        for l in range(LAYERS):
            q, k, v, a, b = self.inputs[l]
            self.lay.step(self.views[l], self.idx, q, k, v, self.outs[l], DK ** -0.5,
                          gate=(a, b, self.A_log, self.dt_bias))

    def prewarm(self, steps, gen):
        """Random steps from the input distributions so that codes, scales and buffers hold realistic values."""
        for t in range(steps):
            if t % 64 == 0:                      # refresh the activations now and then
                self.inputs = [make_inputs(self.batch, gen, self.device) for _ in range(LAYERS)]
            self.step()
        torch.cuda.synchronize()

    def stagger(self):
        """Spread the slots' buffer positions uniformly over the fold period: row r takes r mod m extra tokens (the other
        rows sit out as padding rows), so that afterwards every step folds an m-th of the slots."""
        keep = self.idx
        rows = torch.arange(self.batch, device=self.device) % M
        for j in range(1, M):
            self.idx = torch.where(rows >= j, keep, torch.zeros_like(keep))
            self.step()
        self.idx = keep
        torch.cuda.synchronize()

    def capture(self):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        from statequant_b200 import _cabi
        n0 = _cabi.launch_count()
        with torch.cuda.graph(self.graph):
            self.step()
        self.launches_per_step = _cabi.launch_count() - n0     # kernel nodes of the captured step

    def timed(self, steps):
        """ms for `steps` graph replays, CUDA events on the launching stream."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            if self.graph is not None:
                self.graph.replay()
            else:
                self.step()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)


class Mamba2Stack(Stack):
    """Mamba2 / SSD layers at Nemotron-H shapes (128 heads in 8 groups, head_dim 64, d_state 128), int8 k g32."""
    H, GR, DS, HD = 128, 8, 128, 64

    def __init__(self, preset, batch, device, seed):
        import statequant_b200 as sq
        from statequant_b200.kernels import Mamba2SlotLayout
        fmt = {'int8k': (8, 'k', 32), 'int8k128': (8, 'k', 128), 'pace4': (4, 'k', 64)}[preset]
        self.lay = Mamba2SlotLayout(sq.Quantizer(*fmt), self.H, self.GR, self.DS, self.HD, m=M, buffer_bits=8)
        self.batch, self.device = batch, device
        gen = torch.Generator().manual_seed(seed)
        self.blobs = [self.lay.alloc(batch + 1, device) for _ in range(LAYERS)]
        self.views = [self.lay.views(b) for b in self.blobs]
        self.idx = (torch.randperm(batch, generator=gen) + 1).to(torch.int32).to(device)
        self.inputs = [self.make(batch, gen, device) for _ in range(LAYERS)]
        self.A = (-torch.exp(torch.rand(self.H, generator=gen) * math.log(16.0))).to(device)
        self.D = torch.randn(self.H, generator=gen).to(device)
        self.dt_bias = (torch.rand(self.H, generator=gen) * 2.0 - 4.0).to(device)
        self.outs = [torch.empty(batch, self.H, self.HD, dtype=torch.bfloat16, device=device) for _ in range(LAYERS)]
        self.graph, self.launches_per_step = None, None

    def make(self, batch, gen, device):
        f = lambda *s: torch.randn(*s, generator=gen)                                    # noqa: E731
        return [t.to(device) for t in (f(batch, self.H, self.HD).bfloat16(), f(batch, self.H).bfloat16(),
                                       f(batch, self.GR, self.DS).bfloat16(), f(batch, self.GR, self.DS).bfloat16())]

    def step(self):
        for l in range(LAYERS):
            x, dt, B, C = self.inputs[l]
            self.lay.step(self.views[l], self.idx, x, dt, B, C, self.outs[l], self.A, D=self.D, dt_bias=self.dt_bias)

    def prewarm(self, steps, gen):
        for t in range(steps):
            if t % 64 == 0:
                self.inputs = [self.make(self.batch, gen, self.device) for _ in range(LAYERS)]
            self.step()
        torch.cuda.synchronize()

    def bytes_per_slot(self):
        b, m, L = self.lay.breakdown(), self.lay.m, self.lay
        state = (b['S'] + b.get('SC', 0)) * (1 + 1 / m)
        buf = b['KB'] + b['UB'] + b.get('KBS', 0) + b.get('UBS', 0) + b['GB']
        io = 2 * (2 * self.GR * self.DS + self.H * self.HD + self.H) + 2 * self.H * self.HD
        return state + buf * (m - 1) / (2 * m) + buf / m + 2 * (b['GCUR'] + b['NPTR']) + io, state


class KDAStack(Stack):
    """KDA layers at Kimi-Linear-like shapes (32 heads, d 128), per-channel decays, pace4 state."""
    H = 32

    def __init__(self, preset, batch, device, seed):
        import statequant_b200 as sq
        from statequant_b200.kernels import KDASlotLayout
        self.lay = KDASlotLayout(sq.Quantizer(*PRESETS[preset]), self.H, DK, DV, m=M, buffer_bits=8)
        self.batch, self.device = batch, device
        gen = torch.Generator().manual_seed(seed)
        self.blobs = [self.lay.alloc(batch + 1, device) for _ in range(LAYERS)]
        self.views = [self.lay.views(b) for b in self.blobs]
        self.idx = (torch.randperm(batch, generator=gen) + 1).to(torch.int32).to(device)
        self.inputs = [self.make(batch, gen, device) for _ in range(LAYERS)]
        self.outs = [torch.empty(batch, self.H, DV, dtype=torch.bfloat16, device=device) for _ in range(LAYERS)]
        self.graph, self.launches_per_step = None, None

    def make(self, batch, gen, device):
        f = lambda *s: torch.randn(*s, generator=gen)                                    # noqa: E731
        q, k = f(batch, self.H, DK), f(batch, self.H, DK)
        q, k = q / q.norm(dim=-1, keepdim=True), k / k.norm(dim=-1, keepdim=True)
        g = torch.nn.functional.logsigmoid(f(batch, self.H, DK) + 3.0)
        return [t.to(device) for t in (q.bfloat16(), k.bfloat16(), f(batch, self.H, DV).bfloat16(), g.float(),
                                       torch.sigmoid(f(batch, self.H)).float())]

    def step(self):
        for l in range(LAYERS):
            q, k, v, g, beta = self.inputs[l]
            self.lay.step(self.views[l], self.idx, q, k, v, g, beta, self.outs[l], DK ** -0.5)

    prewarm = Mamba2Stack.prewarm

    def bytes_per_slot(self):
        b, m = self.lay.breakdown(), self.lay.m
        state = (b['S'] + b.get('SC', 0)) * (1 + 1 / m)
        buf = b['KB'] + b['UB'] + b.get('KBS', 0) + b.get('UBS', 0) + b['GB']
        io = 2 * (2 * self.H * DK + self.H * DV) + 4 * (self.H * DK + self.H) + 2 * self.H * DV
        return state + buf * (m - 1) / (2 * m) + buf / m + 2 * (b['GCUR'] + b['NPTR']) + io, state


class GGAStack(Stack):
    """GDN layers on the GGA mixed-width state (per-layer widths 4,6,4,4,6,4 repeating, no pivots) with the
    pure-write window of 8 pairs: the whole head is read, re-fitted and rewritten every token."""

    def __init__(self, preset, batch, device, seed):
        from statequant_b200.kernels import GGAPacked
        from statequant_b200.kernels.gga import StepPlan
        gen = torch.Generator().manual_seed(seed)
        widths = [4, 6, 4, 4, 6, 4]
        plan = StepPlan({l: (torch.full((HV,), widths[l % 6]), torch.rand(HV, DK, generator=gen) + 0.5)
                         for l in range(LAYERS)}, 32, name='bench')
        self.lay = GGAPacked(plan, HV, HK, DK, DV, pw=True, m=M)
        self.batch, self.device = batch, device
        self.blobs = [self.lay.alloc(batch + 1, device) for _ in range(LAYERS)]
        self.views = [self.lay.views(b) for b in self.blobs]
        self.idx = (torch.randperm(batch, generator=gen) + 1).to(torch.int32).to(device)
        self.inputs = [make_inputs(batch, gen, device) for _ in range(LAYERS)]
        self.A_log = (torch.randn(HV, generator=gen) * 0.3).to(device)
        self.dt_bias = torch.randn(HV, generator=gen).to(device)
        self.outs = [torch.empty(batch, HV, DV, dtype=torch.bfloat16, device=device) for _ in range(LAYERS)]
        self.graph, self.launches_per_step = None, None
        self.widths = widths

    def step(self):
        for l in range(LAYERS):
            q, k, v, a, b = self.inputs[l]
            self.lay.step(self.views[l], self.idx, q, k, v, self.outs[l], DK ** -0.5,
                          gate=(a, b, self.A_log, self.dt_bias), layer=l)

    def bytes_per_slot(self):
        # state read + written every token, window read, one pair and the P scales rewritten, bf16 I/O
        per = {4: 691616.0, 6: 953760.0}
        tot = sum(per[self.widths[l % 6]] for l in range(LAYERS)) / LAYERS
        st = sum({4: 557056.0, 6: 819200.0}[self.widths[l % 6]] for l in range(LAYERS)) / LAYERS
        return tot, st


WORKLOADS = {'gdn': Stack, 'mamba2': Mamba2Stack, 'kda': KDAStack, 'gga': GGAStack}
WORKLOAD_TEXT = {
    'mamba2': 'Mamba2 / SSD decode stack, Nemotron-H shapes (128 heads in 8 groups, head_dim 64, d_state 128, m 8, int8 buffer)',
    'kda': 'KDA decode stack, Kimi-Linear-like shapes (32 heads, d 128, per-channel decays, m 8, int8 buffer)',
    'gga': 'GDN decode stack on the GGA mixed-width state (widths 4,6,4,4,6,4 repeating) with the pure-write window (8 pairs)',
}


def _arena(tensors, device, pinned=False):
    """One flat byte buffer holding copies of `tensors` (256-byte aligned), and typed views of it in the same order."""
    offs, total = [], 0
    for t in tensors:
        offs.append(total)
        total += (t.numel() * t.element_size() + 255) // 256 * 256
    buf = torch.empty(total, dtype=torch.uint8, device=device)
    if pinned:
        buf = buf.pin_memory()
    views = []
    for t, o in zip(tensors, offs):
        v = buf[o:o + t.numel() * t.element_size()].view(t.dtype).view(t.shape)
        v.copy_(t)
        views.append(v)
    return buf, views


def run_e2e(stack, steps, warmup):
    """The same stack driven through the public API from HOST buffers.  Every step copies that step's activations for
    all layers from pinned host memory (one flat buffer, one copy), launches the 24 layer steps, and reads the last
    layer's output back.  The device side keeps two input buffers, each with its own captured step, so that the copy
    of step t + 1 runs on a second stream while step t computes; every step's copy and read-back are inside the timed
    region."""
    flat = [t for lay_in in stack.inputs for t in lay_in]
    sizes = [len(lay_in) for lay_in in stack.inputs]
    host_buf, _ = _arena(flat, 'cpu', pinned=True)
    out_h = torch.empty_like(stack.outs[-1], device='cpu').pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in flat)
    d2h = out_h.numel() * out_h.element_size()

    bufs, graphs = [], []
    for _ in range(2):
        dbuf, views = _arena(flat, stack.device)
        it = iter(views)
        stack.inputs = [[next(it) for _ in range(n)] for n in sizes]
        stack.capture()
        bufs.append(dbuf)
        graphs.append(stack.graph)
    main, side = torch.cuda.current_stream(), torch.cuda.Stream()
    copied = [torch.cuda.Event() for _ in range(2)]
    used = [torch.cuda.Event() for _ in range(2)]
    for e in used:
        e.record(main)

    def one(t):
        i = t & 1
        side.wait_event(used[i])                       # the step that last read this buffer has finished
        with torch.cuda.stream(side):
            bufs[i].copy_(host_buf, non_blocking=True)
            copied[i].record(side)
        main.wait_event(copied[i])
        graphs[i].replay()
        used[i].record(main)
        out_h.copy_(stack.outs[-1], non_blocking=True)

    for t in range(warmup):
        one(t)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for t in range(steps):
        one(warmup + t)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1), h2d, d2h


def cpu_baseline(batch, steps, warmup, preset='int8k'):
    """The oracle (CPU restatement of the reference's torch path) on one layer, all host threads: layer-steps/s."""
    import statequant_b200 as sq
    from oracle import oracle
    from statequant_b200.kernels import SlotLayout
    lay = SlotLayout(sq.Quantizer(*PRESETS[preset]), HV, HK, DK, DV, m=M, buffer_bits=8)
    gen = torch.Generator().manual_seed(7)
    blob = lay.alloc(batch + 1, 'cpu')
    V = lay.views(blob)
    lay.write(V, torch.arange(1, batch + 1), torch.randn(batch, HV, DV, DK, generator=gen) * 0.3)
    idx = torch.arange(1, batch + 1, dtype=torch.int32)
    q, k, v, a, b = make_inputs(batch, gen, 'cpu')
    A_log, dtb = torch.randn(HV, generator=gen) * 0.3, torch.randn(HV, generator=gen)
    out = torch.empty(batch, HV, DV, dtype=torch.bfloat16)
    oracle.set_num_threads(os.cpu_count() or 1)        # all host cores, whatever OMP_NUM_THREADS a launcher exported
    for _ in range(warmup):
        oracle.gdn_step(lay, V, idx, q, k, v, out, DK ** -0.5, gate=(a, b, A_log, dtb))
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.gdn_step(lay, V, idx, q, k, v, out, DK ** -0.5, gate=(a, b, A_log, dtb))
    dt = time.perf_counter() - t0
    return steps / dt, oracle.num_threads(), dt


def time_slot_io(preset, batch, device, layers=4, reps=5):
    """The prefill boundary of the same layout (the device kernels behind ``SlotLayout.read`` / ``write``): one call
    reads `batch` slots' current state as fp32 (stored state advanced across the pending buffer), one call packs fp32
    states into the slots.  Rotating over `layers` blobs (far above L2), CUDA events, microseconds per call and
    algorithmic GB/s (fp32 states + the slots' packed bytes)."""
    import statequant_b200 as sq
    from statequant_b200.kernels import SlotLayout
    lay = SlotLayout(sq.Quantizer(*{**PRESETS, **EXTRA_PRESETS}[preset]), HV, HK, DK, DV, m=M, buffer_bits=8)
    gen = torch.Generator().manual_seed(3)
    blobs = [lay.alloc(batch + 1, device) for _ in range(layers)]
    views = [lay.views(b) for b in blobs]
    idx = (torch.randperm(batch, generator=gen) + 1).to(torch.int32).to(device)
    S = [(torch.randn(batch, HV, DV, DK, generator=gen) * 0.3).to(device) for _ in range(2)]
    for v in views:
        lay.write(v, idx, S[0])
    bd = lay.breakdown()
    packed = bd['S'] + bd.get('SC', 0)
    f32 = HV * DV * DK * 4
    out = {}
    for name, fn, nbytes in (('write', lambda v, i: lay.write(v, idx, S[i & 1]), f32 + packed),
                             ('read', lambda v, i: lay.read(v, idx), f32 + packed + bd['KB'] + bd['UB'])):
        for i, v in enumerate(views):
            fn(v, i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for r in range(reps):
            for i, v in enumerate(views):
                fn(v, i)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * layers)
        out[name + '_us_per_call'] = us
        out[name + '_gbs'] = batch * nbytes / (us * 1e-6) / 1e9
    out['slots_per_call'] = batch
    out['workload'] = f'SlotLayout.read / write of {batch} slots ({preset}), fp32 states in HBM'
    return out


def time_conv_update(batch, device, layers=24, reps=6):
    """The short causal convolution in front of the step (`causal_conv1d_update`, one token per row): the GDN layer's
    mixed q | k | v row of 2 HK DK + HV DV channels, width 4, bf16, SiLU, the cache as vLLM lays it out
    ([lines, 3, dim]).  One cache per layer (24 x 12.6 MB: above L2), a CUDA graph of one call per layer, CUDA events.
    Algorithmic bytes per row and channel: 3 state elements read and written, x read, the result written."""
    from statequant_b200.kernels import causal_conv1d_update
    gen = torch.Generator().manual_seed(5)
    dim, width = 2 * HK * DK + HV * DV, 4
    caches = [torch.randn(batch + 1, width - 1, dim, generator=gen).to(torch.bfloat16).to(device) for _ in range(layers)]
    xs = [torch.randn(batch, dim, generator=gen).to(torch.bfloat16).to(device) for _ in range(layers)]
    w = (torch.randn(dim, width, generator=gen) * 0.5).to(torch.bfloat16).to(device)
    b = (torch.randn(dim, generator=gen) * 0.1).to(torch.bfloat16).to(device)
    idx = (torch.randperm(batch, generator=gen) + 1).to(torch.int32).to(device)

    def step():
        for c, x in zip(caches, xs):
            causal_conv1d_update(x, c.transpose(1, 2), w, b, 'silu', idx)

    step()
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        step()
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        gr.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * layers)
    nbytes = batch * dim * 2 * (2 * (width - 1) + 2)
    peak, _ = measured_peak_gbs()
    return {'us_per_call': us, 'gbs': nbytes / (us * 1e-6) / 1e9, 'frac_of_peak': nbytes / (us * 1e-6) / 1e9 / peak,
            'algorithmic_bytes_per_call': nbytes, 'rows': batch, 'dim': dim,
            'workload': f'causal_conv1d_update, {batch} rows x {dim} channels, width {width}, bf16, SiLU, {layers} caches in rotation'}


def ncu_traffic(preset, batch):
    """DRAM bytes (read + write) per layer-step from the ncu captures summarised under profiles/ (traffic.json, written
    next to the summaries: per preset the bytes of a launch that does not fold and of one in which every head folds,
    at batch 256); averaged over the fold period and scaled to the batch (traffic grows in proportion to it)."""
    try:
        t = json.load(open(os.path.join(ROOT, 'profiles', 'traffic.json')))[preset]
        return (t['step_bytes'] * (M - 1) + t['fold_step_bytes']) / M * batch / t.get('batch', 256)
    except Exception:
        return None


def run_config4(args, rank, world, device, barrier, max_over_ranks, table=8192, batches=(64, 256, 1024, 4096), layers=4):
    """The slot-scaling sweep: one GDN layer stack on the GGA mixed-width state (per-layer widths 4,6,4,4,6,... with the
    pure-write window), a state table of `table` slots, and ONE global batch of 64 / 256 / 1024 / 4096 rows drawn as
    the prefix of a seeded random permutation of slots 1 .. table - 1 (slot 0 is padding).  On N GPUs the table is
    sharded (slot s lives on rank (s - 1) mod N, statequant_b200/sharding.py), every rank serves the rows whose
    slots it owns, and the time of a layer-step is the slowest rank's: strong scaling, with the imbalance of a
    random batch across the shards reported next to it.  No collective on the data path."""
    global LAYERS
    from statequant_b200 import sharding
    from statequant_b200.kernels import GGAPacked
    from statequant_b200.kernels.gga import StepPlan
    gen = torch.Generator().manual_seed(99)                        # the same on every rank
    widths = [4, 6, 4, 4, 6, 4]
    plan = StepPlan({l: (torch.full((HV,), widths[l % 6]), torch.rand(HV, DK, generator=gen) + 0.5) for l in range(layers)},
                    32, name='config4')
    lay = GGAPacked(plan, HV, HK, DK, DV, pw=True, m=M)
    nloc = sharding.local_slots(table, rank, world)
    blobs = [lay.alloc(nloc, device) for _ in range(layers)]
    views = [lay.views(b) for b in blobs]
    perm = torch.randperm(table - 1, generator=gen) + 1
    A_log, dtb = (torch.randn(HV, generator=gen) * 0.3).to(device), torch.randn(HV, generator=gen).to(device)
    out = {'table_slots': table, 'layers': layers, 'slot_bytes': lay.nbytes, 'scaling': 'strong', 'batches': {}}
    for B in batches:
        gidx = perm[:B].to(torch.int32)
        rows = sharding.rows_of(gidx, rank, world)
        lidx = sharding.to_local(gidx, rank, world)[rows].contiguous().to(device)
        nb = int(rows.numel())
        ins = [make_inputs(max(nb, 1), gen, device) for _ in range(layers)]
        outs = [torch.empty(max(nb, 1), HV, DV, dtype=torch.bfloat16, device=device) for _ in range(layers)]

        def step():
            if nb:
                for l in range(layers):
                    q, k, v, a, b = ins[l]
                    lay.step(views[l], lidx, q, k, v, outs[l], DK ** -0.5, gate=(a, b, A_log, dtb), layer=l)
        for _ in range(3):
            step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        nrep = 4
        e0.record()
        for _ in range(nrep):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1))
        most = max_over_ranks(float(nb))
        out['batches'][str(B)] = {'us_per_layer_step': ms * 1e3 / (nrep * layers), 'rows_on_busiest_rank': int(most),
                                  'imbalance': most * world / B}
    del blobs, views
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=128)
    ap.add_argument('--warmup', type=int, default=8)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--batch', type=int, default=256)
    ap.add_argument('--prewarm', type=int, default=512)
    ap.add_argument('--preset', default='int8k', choices=list(PRESETS) + list(EXTRA_PRESETS) + ['int8k128'])
    ap.add_argument('--no-variants', action='store_true', help='time the headline preset only')
    ap.add_argument('--layers', type=int, default=24, help='layers of the stack (24 = the benchmark; fewer for ncu captures)')
    ap.add_argument('--no-e2e', action='store_true', help='skip the host-buffer leg')
    ap.add_argument('--no-cpu', action='store_true', help='skip the CPU-baseline leg')
    ap.add_argument('--eager', action='store_true', help='launch eagerly instead of replaying a CUDA graph')
    ap.add_argument('--workload', default='gdn', choices=list(WORKLOADS),
                    help='gdn = the benchmark; mamba2 / kda / gga time the other kernel families on their shapes')
    ap.add_argument('--mma-hpc', type=int, default=0, help='tensor-core kernels: value heads per CTA (0: a whole key head)')
    ap.add_argument('--kernel-path', type=int, default=0, choices=[0, 1, 2, 3, 4],
                    help='0 best kernel for the shape; 1 generic; 2 staged + fold launch (profiling / comparison)')
    ap.add_argument('--conv-only', action='store_true',
                    help='time only the causal conv update in front of the step (--layers caches in rotation) and print its figures')
    args = ap.parse_args()
    global LAYERS
    LAYERS = args.layers
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    config = {'workload': f'24-layer GDN decode stack, Qwen3.5-4B shapes (HV 32, HK 16, d 128, m 8, int8 buffer), '
                          f'state preset {args.preset}, batch {args.batch} slots per GPU, bf16 activations, in-kernel gate',
              'layers': LAYERS, 'batch_per_gpu': args.batch, 'preset': args.preset, 'prewarm_steps': args.prewarm,
              'l2': 'working set per step (all layers) far exceeds L2; no flush needed',
              'sharding': 'slots sharded across GPUs, no collective'}

    if args.impl == 'reference':
        if rank != 0:
            return
        from oracle import oracle
        oracle.build()                                        # the CPU oracle only: this arm loads no CUDA library
        steps = max(1, args.steps)
        val, cores, dt = cpu_baseline(args.batch, steps, max(1, min(args.warmup, 8)), args.preset)
        sample = f'one layer of the stack, batch {args.batch}, {steps} layer-steps, {dt:.1f} s wall'
        print(json.dumps({
            'impl': 'reference', 'metric': METRIC, 'value': val, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': steps,
            'warmup': args.warmup, 'ms_per_step': 1e3 / val, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic', 'config': config,
            'cpu_baseline': {'value': val, 'unit': UNIT, 'cores': cores, 'kind': 'port', 'sample': sample},
            'e2e': {'value': val, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}))
        return

    from statequant_b200 import _cabi
    assert torch.cuda.is_available(), 'bench.py needs a GPU (there is no CPU fallback)'
    torch.cuda.set_device(local)
    _cabi.set_option('kernel_path', args.kernel_path)
    if args.mma_hpc:
        _cabi.set_option('mma_heads_per_cta', args.mma_hpc)
    device = f'cuda:{local}'
    if args.conv_only:
        if rank == 0:
            print(json.dumps({'conv_update': time_conv_update(args.batch, device, layers=args.layers, reps=max(1, args.steps))}))
        return
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=torch.device(device))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    results = {}
    if args.workload != 'gdn':
        args.no_variants, args.no_e2e, args.no_cpu = True, True, True
        config['workload'] = (f'{WORKLOAD_TEXT[args.workload]}, state preset {args.preset}, batch {args.batch} slots per '
                              f'GPU, bf16 activations')
    presets = [args.preset] + ([] if args.no_variants else [p for p in PRESETS if p != args.preset])
    # The state is folded every M = 8 tokens and a fold step costs several plain steps, so only whole fold periods are
    # timed: the requested step count is rounded up to a multiple of 8.
    steps_timed = -(-args.steps // M) * M
    config['fold_period_steps'] = M
    config['steps_timed'] = steps_timed
    clocks = None
    launches = 0
    e2e = None

    def time_stack(stack, steps, sample_clocks=False, stagger=False):
        stack.prewarm(args.prewarm, torch.Generator().manual_seed(4321 + rank))
        if stagger:
            stack.stagger()
        if not args.eager:
            stack.capture()
        stack.timed(max(3, args.warmup))
        barrier()
        sampler = ClockSampler(local) if (sample_clocks and rank == 0) else None
        t0 = time.time()
        l0 = _cabi.launch_count()
        ms = stack.timed(steps)
        barrier()
        t1 = time.time()
        ms = max_over_ranks(ms)
        clk = sampler.stop(t0, t1) if sampler is not None else None
        total, state = stack.bytes_per_slot()
        lsteps = steps * LAYERS
        per_launch_s = ms * 1e-3 / lsteps
        res = {'layer_steps_per_s': world * lsteps / (ms * 1e-3), 'us_per_layer_step': per_launch_s * 1e6,
               'ms_per_step': ms / steps, 'layers': LAYERS, 'steps_timed': steps,
               'total_gbs_per_gpu': args.batch * total / per_launch_s / 1e9,
               'state_gbs_per_gpu': args.batch * state / per_launch_s / 1e9,
               'bytes_per_slot_layer_step': total}
        nl = (stack.launches_per_step * steps if stack.launches_per_step is not None else _cabi.launch_count() - l0)
        return res, clk, nl

    for pi, preset in enumerate(presets):
        stack = WORKLOADS[args.workload](preset, args.batch, device, seed=1234 + rank)
        res, clk, nl = time_stack(stack, steps_timed, sample_clocks=pi == 0)
        results[preset] = res
        if pi == 0:
            clocks, launches = clk, nl
        if pi == 0 and not args.no_e2e and not args.eager:
            barrier()
            esteps = max(M, min(steps_timed, 32))
            ems, h2d, d2h = run_e2e(stack, esteps, 3)
            ems = max_over_ranks(ems)
            e2e = {'value': world * esteps * LAYERS / (ems * 1e-3), 'unit': UNIT, 'h2d_bytes_per_step': h2d,
                   'd2h_bytes_per_step': d2h, 'steps': esteps,
                   'note': 'per step: all 24 layers\' activations copied from pinned host memory (one copy, on a second stream, '
                           'overlapping the previous step), last layer\'s output read back'}
        del stack
        torch.cuda.empty_cache()

    if args.workload == 'gdn' and not args.no_variants:
        # the other kernel families on their own shapes (8-layer stacks: far above L2), and the slot-scaling sweep
        saved = LAYERS
        LAYERS = min(8, saved)
        for name, wl, preset in (('mamba2_int8k', 'mamba2', 'int8k'), ('kda_pace4', 'kda', 'pace4'), ('gga_pw', 'gga', 'pace4')):
            stack = WORKLOADS[wl](preset, args.batch, device, seed=1234 + rank)
            keep = args.prewarm
            args.prewarm = min(args.prewarm, 64)
            res, _, _ = time_stack(stack, max(M, min(steps_timed, 32)))
            args.prewarm = keep
            res['workload'] = WORKLOAD_TEXT[wl]
            results[name] = res
            del stack
            torch.cuda.empty_cache()
        # the headline stack with the slots at different buffer positions, as a serving engine has them (the
        # headline itself keeps the baseline's protocol: all slots in lockstep, one step in eight folds everything)
        stack = WORKLOADS['gdn'](args.preset, args.batch, device, seed=1234 + rank)
        keep = args.prewarm
        args.prewarm = min(args.prewarm, 64)
        res, _, _ = time_stack(stack, max(M, min(steps_timed, 32)), stagger=True)
        args.prewarm = keep
        res['workload'] = 'the headline stack (8 layers) with the slots\' buffer positions spread uniformly over the fold period'
        results[args.preset + '_staggered'] = res
        del stack
        torch.cuda.empty_cache()
        # the same with the fold as its own, balanced launch behind a step kernel that only appends (kernel_path 3):
        # what an engine whose slots sit at different buffer positions should select
        _cabi.set_option('kernel_path', 3)
        stack = WORKLOADS['gdn'](args.preset, args.batch, device, seed=1234 + rank)
        args.prewarm = min(args.prewarm, 64)
        res, _, _ = time_stack(stack, max(M, min(steps_timed, 32)), stagger=True)
        args.prewarm = keep
        _cabi.set_option('kernel_path', args.kernel_path)
        res['workload'] = 'the staggered stack with kernel_path 3: tensor-core step kernel that only appends + the fold launch'
        results[args.preset + '_staggered_fold_launch'] = res
        del stack
        torch.cuda.empty_cache()
        LAYERS = saved
        results['slot_io_' + args.preset] = time_slot_io(args.preset, args.batch, device)
        results['conv_update'] = time_conv_update(args.batch, device)
        results['config4_gga_slot_scaling'] = run_config4(args, rank, world, device, barrier, max_over_ranks)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    head = results[args.preset]
    peak, which = measured_peak_gbs()
    line = {
        'metric': METRIC if args.workload == 'gdn' else f'decode layer-steps/s ({args.workload} stack)', 'value': head['layer_steps_per_s'], 'unit': UNIT, 'n_gpus': world, 'steps': args.steps, 'steps_timed': steps_timed,
        'warmup': max(3, args.warmup), 'ms_per_step': head['ms_per_step'], 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic', 'config': config,
        'us_per_layer_step': head['us_per_layer_step'],
        'state_gbs_per_gpu': head['state_gbs_per_gpu'], 'state_frac_of_8tbs': head['state_gbs_per_gpu'] / 8000.0,
        'total_frac_of_8tbs': head['total_gbs_per_gpu'] / 8000.0,
        'roofline': {'bound': 'hbm', 'achieved': head['total_gbs_per_gpu'], 'peak': peak, 'unit': 'GB/s',
                     'frac': head['total_gbs_per_gpu'] / peak, 'traffic': ncu_traffic(args.preset, args.batch) if args.workload == 'gdn' else None,
                     'peak_source': which,
                     'kernel': 'step_mma_kernel<GDN>: the one launch of a layer-step (one C-ABI call; on a slot\'s 8th token it '
                               'also folds), averaged over whole fold periods of 8 steps',
                     'algorithmic_bytes_per_launch': args.batch * head['bytes_per_slot_layer_step']},
        'variants': results, 'clocks': clocks, 'e2e': e2e, 'gpu_launches': launches,
    }
    if world == 1 and not args.no_cpu:
        from oracle import oracle
        oracle.build()
        v, cores, dt = cpu_baseline(args.batch, 16, 4, args.preset)
        line['cpu_baseline'] = {'value': v, 'unit': UNIT, 'cores': cores, 'kind': 'port',
                                'sample': f'one layer of the stack, batch {args.batch}, 16 layer-steps after 4 warm-up, {dt:.1f} s wall'}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
