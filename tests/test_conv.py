"""The short causal convolution in front of the decode step.

CPU: the oracle (oracle/sq_oracle_conv.c) against a plain torch statement of the op, argument checks of the C ABI.
GPU: the CUDA kernels against the oracle on the same bytes (conv state byte for byte, outputs to the last bit of the
storage type up to rare exp / division ulps), every layout and type the launcher dispatches on, and against vLLM's
own Triton kernel -- the op the reference's forward calls (src/statequant/integrations/vllm_plugin.py:379-381).
"""
import ctypes as C

import pytest
import torch

from oracle import oracle
from statequant_b200 import _cabi

DT = {'bf16': torch.bfloat16, 'f16': torch.float16, 'f32': torch.float32}


def make_case(rows, dim, width, state_len, xdt, wdt, layout, lines=None, seed=0, bias=True, pad_rows=True):
    """Seeded inputs on the host.  layout 'tok_dim': the cache is [lines, state_len, dim] and the op sees its
    transposed view (vLLM's default); 'dim_tok': the cache is [lines, dim, state_len]."""
    g = torch.Generator().manual_seed(1234 + seed)
    lines = lines or rows + 3
    x = torch.randn(rows, dim, generator=g).to(xdt)
    if layout == 'tok_dim':
        cache = torch.randn(lines, state_len, dim, generator=g).to(xdt)
        state = cache.transpose(1, 2)
    else:
        cache = torch.randn(lines, dim, state_len, generator=g).to(xdt)
        state = cache
    w = (torch.randn(dim, width, generator=g) * 0.5).to(wdt)
    b = (torch.randn(dim, generator=g) * 0.1).to(wdt) if bias else None
    idx = torch.randperm(lines - 1, generator=g)[:rows].to(torch.int32) + 1          # distinct lines, none the null block
    if pad_rows and rows >= 4:
        idx[1] = 0                                                                     # null block
        idx[rows - 1] = -1                                                             # PAD_SLOT_ID
    return x, cache, state, w, b, idx


def torch_statement(x, state, w, b, silu, idx, null=0):
    """The op in plain torch, one row at a time (typed products as torch's own 16-bit multiply)."""
    x, state = x.clone(), state.clone()
    width, state_len = w.size(1), state.size(2)
    typed = x.dtype != torch.float32 and w.dtype == x.dtype
    for r in range(x.size(0)):
        line = r if idx is None else int(idx[r])
        if line < 0 or line == null:
            continue
        xn = x[r].clone()
        acc = b.float().clone() if b is not None else torch.zeros(x.size(1))
        for j in range(width):
            col = xn if j == width - 1 else state[line, :, j]
            if typed:
                acc = acc + (col * w[:, j]).float()
            else:                                   # fused product: exact in double, one rounding with the sum
                acc = (col.double() * w[:, j].double() + acc.double()).float()
        state[line, :, :state_len - 1] = state[line, :, 1:].clone()
        state[line, :, state_len - 1] = xn
        if silu:
            acc = acc / (1.0 + torch.exp(-acc))
        x[r] = acc.to(x.dtype)
    return x, state


def close_in_storage_type(a, b, frac=2e-3):
    """Equal to within one unit in the last place of the storage type, and different in few places at all."""
    if a.dtype == torch.float32:
        torch.testing.assert_close(a, b, rtol=2e-6, atol=1e-7)
        return
    ia, ib = a.view(torch.int16).int(), b.view(torch.int16).int()
    d = (ia - ib).abs()
    assert int(d.max()) <= 1, f'outputs differ by {int(d.max())} units in the last place'
    assert float((d > 0).float().mean()) <= frac, f'{float((d > 0).float().mean()):.2e} of the outputs differ'


CASES = [
    # rows, dim, width, state_len, x, w, layout, bias, silu
    (6, 64, 4, 3, 'bf16', 'bf16', 'tok_dim', True, True),
    (6, 64, 4, 3, 'bf16', 'bf16', 'dim_tok', True, True),
    (5, 48, 3, 2, 'f16', 'f16', 'tok_dim', True, True),
    (5, 48, 2, 1, 'f32', 'f32', 'dim_tok', False, False),
    (4, 40, 4, 5, 'bf16', 'bf16', 'tok_dim', True, True),        # a line longer than the window
    (4, 40, 4, 3, 'bf16', 'f32', 'dim_tok', True, True),         # 16-bit activations, fp32 taps
    (4, 36, 3, 2, 'f32', 'bf16', 'tok_dim', True, False),
]


@pytest.mark.parametrize('case', CASES, ids=lambda c: '-'.join(map(str, c)))
def test_oracle_matches_torch_statement(case):
    rows, dim, width, sl, xd, wd, layout, bias, silu = case
    x, cache, state, w, b, idx = make_case(rows, dim, width, sl, DT[xd], DT[wd], layout, bias=bias)
    want_x, want_state = torch_statement(x, state, w, b, silu, idx)
    cache0 = cache.clone()
    got = oracle.conv1d_update(x, state, w, b, 'silu' if silu else None, idx)
    assert torch.equal(state, want_state)
    close_in_storage_type(got, want_x)
    # padding rows: neither the row nor any cache line it could name was touched
    if rows >= 4:
        assert torch.equal(cache[0], cache0[0])


def test_oracle_without_indices_uses_the_row_as_line():
    x, cache, state, w, b, _ = make_case(3, 32, 4, 3, torch.bfloat16, torch.bfloat16, 'tok_dim', lines=3)
    want_x, want_state = torch_statement(x, state, w, b, True, None, null=-1)
    oracle.conv1d_update(x, state, w, b, True, None, null_block_id=None)
    assert torch.equal(state, want_state)
    close_in_storage_type(x, want_x)


def test_struct_size_and_bad_arguments():
    import os
    import subprocess
    import tempfile
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = '#include <stdio.h>\n#include "statequant_b200.h"\nint main(){printf("%zu", sizeof(sqb_conv_update_t));return 0;}'
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, 't.c'), 'w').write(src)
        subprocess.run(['gcc', '-I', os.path.join(root, 'include'), os.path.join(d, 't.c'), '-o', os.path.join(d, 't')], check=True)
        assert int(subprocess.run([os.path.join(d, 't')], capture_output=True, text=True).stdout) == C.sizeof(_cabi.ConvUpdate)
    L = _cabi.lib()
    a = _cabi.ConvUpdate(rows=2, dim=64, width=4, state_len=3)
    assert L.sqb_conv1d_update(C.byref(a), None) == -1 and b'NULL' in L.sqb_last_error()
    buf = (C.c_char * 64)()
    p = C.addressof(buf)
    a = _cabi.ConvUpdate(x=p, out=p, state=p, w=p, rows=2, dim=64, width=5, state_len=4)
    assert L.sqb_conv1d_update(C.byref(a), None) == -1 and b'width 5' in L.sqb_last_error()
    a.width, a.state_len = 4, 2
    assert L.sqb_conv1d_update(C.byref(a), None) == -1 and b'state_len' in L.sqb_last_error()
    a.state_len, a.x_dtype, a.w_dtype = 3, _cabi.SQB_BF16, _cabi.SQB_F16
    assert L.sqb_conv1d_update(C.byref(a), None) == -1 and b'16-bit' in L.sqb_last_error()
    a.rows = 0
    assert L.sqb_conv1d_update(C.byref(a), None) == 0


# ---- GPU ----------------------------------------------------------------------------------------------------------

GPU_CASES = [
    # rows, dim, width, state_len, x, w, layout, bias, silu          (the vector kernels unless noted)
    (9, 8192, 4, 3, 'bf16', 'bf16', 'tok_dim', True, True),           # GDN of the benchmark, vLLM's cache layout
    (9, 8192, 4, 3, 'bf16', 'bf16', 'dim_tok', True, True),
    (7, 1024, 4, 3, 'f16', 'f16', 'tok_dim', True, True),
    (7, 1024, 3, 2, 'bf16', 'bf16', 'dim_tok', False, True),
    (7, 1024, 2, 1, 'bf16', 'bf16', 'tok_dim', True, False),
    (5, 512, 4, 3, 'f32', 'f32', 'tok_dim', True, True),
    (5, 512, 4, 3, 'f32', 'f32', 'dim_tok', True, True),
    (5, 512, 4, 3, 'bf16', 'f32', 'tok_dim', True, True),
    (5, 512, 3, 2, 'f32', 'bf16', 'dim_tok', True, True),
    (5, 520, 4, 5, 'bf16', 'bf16', 'tok_dim', True, True),            # longer line: the strided kernel
    (5, 100, 4, 3, 'bf16', 'bf16', 'tok_dim', True, True),            # dim not a multiple of 8: the strided kernel
]


@pytest.mark.gpu
@pytest.mark.parametrize('case', GPU_CASES, ids=lambda c: '-'.join(map(str, c)))
def test_cuda_matches_oracle(case):
    from statequant_b200.kernels import causal_conv1d_update
    rows, dim, width, sl, xd, wd, layout, bias, silu = case
    x, cache, state, w, b, idx = make_case(rows, dim, width, sl, DT[xd], DT[wd], layout, bias=bias, seed=3)
    dev = 'cuda:0'
    xg, cg, wg = x.to(dev), cache.to(dev), w.to(dev)
    sg = cg.transpose(1, 2) if layout == 'tok_dim' else cg
    bg = b.to(dev) if b is not None else None
    n0 = _cabi.launch_count()
    for step in range(3):                                  # three tokens: the state moves through the whole window
        out = causal_conv1d_update(xg, sg, wg, bg, 'silu' if silu else None, idx.to(dev))
        assert out.data_ptr() == xg.data_ptr()
        oracle.conv1d_update(x, state, w, b, silu, idx)
        assert torch.equal(cg.cpu(), cache), f'conv state differs after token {step}'
        close_in_storage_type(xg.cpu(), x)
        xg.copy_(x)                                        # the next token's input: the same bits on both sides
    assert _cabi.launch_count() == n0 + 3


@pytest.mark.gpu
def test_cuda_strided_rows_and_graph_replay():
    """x as rows of a wider buffer (row stride > dim), captured once and replayed with other cache lines."""
    from statequant_b200.kernels import causal_conv1d_update
    dev = 'cuda:0'
    rows, dim = 6, 2048
    x, cache, state, w, b, idx = make_case(rows, dim, 4, 3, torch.bfloat16, torch.bfloat16, 'tok_dim', lines=20, seed=5)
    wide = torch.zeros(rows, dim + 256, dtype=torch.bfloat16, device=dev)
    xg = wide[:, :dim]
    cg, wg, bg, ig = cache.to(dev), w.to(dev), b.to(dev), idx.to(dev)
    sg = cg.transpose(1, 2)
    xg.copy_(x)
    causal_conv1d_update(xg, sg, wg, bg, True, ig)         # warm-up outside the capture
    oracle.conv1d_update(x, state, w, b, True, idx)
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        causal_conv1d_update(xg, sg, wg, bg, True, ig)
    for rep in range(3):
        g = torch.Generator().manual_seed(50 + rep)
        idx = torch.randperm(19, generator=g)[:rows].to(torch.int32) + 1
        x = torch.randn(rows, dim, generator=g).to(torch.bfloat16)
        ig.copy_(idx)
        xg.copy_(x)
        gr.replay()
        oracle.conv1d_update(x, state, w, b, True, idx)
        assert torch.equal(cg.cpu(), cache)
        close_in_storage_type(xg.cpu(), x)
    assert float(wide[:, dim:].abs().max()) == 0.0          # nothing past the rows' end was written


@pytest.mark.gpu
def test_conv_then_step_reads_the_slices_in_place():
    """The convolved row is q | k | v: the decode step takes the three column slices as they lie."""
    import statequant_b200 as sq
    from statequant_b200.kernels import SlotLayout, causal_conv1d_update, split_qkv
    dev = 'cuda:0'
    hv, hk, dk, dv, rows = 4, 2, 128, 128, 5
    dim = 2 * hk * dk + hv * dv
    lay = SlotLayout(sq.Quantizer(8, 'k', 32), hv, hk, dk, dv, m=8, buffer_bits=8)
    g = torch.Generator().manual_seed(11)
    blob = lay.alloc(rows + 1, dev)
    V = lay.views(blob)
    lay.write(V, torch.arange(1, rows + 1, device=dev), (torch.randn(rows, hv, dv, dk, generator=g) * 0.3).to(dev))
    idx = torch.arange(1, rows + 1, dtype=torch.int32, device=dev)
    mixed = torch.randn(rows, dim, generator=g).to(torch.bfloat16).to(dev)
    cache = torch.randn(rows + 1, 3, dim, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn(dim, 4, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    x = causal_conv1d_update(mixed, cache.transpose(1, 2), w, None, 'silu', idx)
    q, k, v = split_qkv(x, hk, dk, hv, dv)
    a, b = torch.randn(rows, hv, generator=g).to(torch.bfloat16).to(dev), torch.randn(rows, hv, generator=g).to(torch.bfloat16).to(dev)
    A_log, dtb = (torch.randn(hv, generator=g) * 0.3).to(dev), torch.randn(hv, generator=g).to(dev)
    out = torch.empty(rows, hv, dv, dtype=torch.bfloat16, device=dev)
    out2 = torch.empty_like(out)
    blob2 = blob.clone()
    lay.step(V, idx, q, k, v, out, dk ** -0.5, gate=(a, b, A_log, dtb))
    lay.step(lay.views(blob2), idx, q.contiguous(), k.contiguous(), v.contiguous(), out2, dk ** -0.5, gate=(a, b, A_log, dtb))
    assert torch.equal(out, out2) and torch.equal(blob, blob2)


@pytest.mark.gpu
def test_cuda_matches_vllm_kernel():
    """Against the op the reference's forward calls: vLLM's Triton `causal_conv1d_update`, same inputs, on this GPU.
    The conv state must be the same bytes; the outputs may differ in the last bit of bf16 where Triton's approximate
    exp and division land on the other side of a rounding boundary."""
    try:
        from vllm.model_executor.layers.mamba.ops.causal_conv1d import causal_conv1d_update as vllm_update
    except Exception as err:                                # vLLM absent or not importable on this box
        pytest.skip(f'vLLM op not importable: {err!r}')
    from statequant_b200.kernels import causal_conv1d_update
    dev = 'cuda:0'
    for layout, xdt in (('tok_dim', torch.bfloat16), ('dim_tok', torch.bfloat16), ('tok_dim', torch.float16)):
        rows, dim = 33, 8192
        x, cache, state, w, b, idx = make_case(rows, dim, 4, 3, xdt, xdt, layout, lines=64, seed=9)
        idx = idx.clamp_min(0)                              # vLLM's kernel knows the null block only
        mine_x, mine_c = x.to(dev), cache.to(dev)
        ref_x, ref_c = x.to(dev), cache.to(dev)
        view = (lambda c: c.transpose(1, 2)) if layout == 'tok_dim' else (lambda c: c)
        wg, bg, ig = w.to(dev), b.to(dev), idx.to(dev)
        for _ in range(3):
            try:
                ref_out = vllm_update(ref_x, view(ref_c), wg, bg, 'silu', conv_state_indices=ig)
            except Exception as err:                        # Triton could not build the kernel here
                pytest.skip(f'vLLM op did not run: {err!r}')
            out = causal_conv1d_update(mine_x, view(mine_c), wg, bg, 'silu', ig)
            assert torch.equal(mine_c, ref_c)
            close_in_storage_type(out.cpu(), ref_out.cpu(), frac=5e-3)
            mine_x.copy_(ref_out)
            ref_x.copy_(ref_out)
