"""Drop-in against the REAL reference package: ``binding.bind_reference()`` rebinds an installed / checked-out
``statequant`` onto this package's classes, after which

* (CPU) the reference's own vLLM calculator tests for Gated DeltaNet and Mamba2 pass on the rebound layouts
  (reference: tests/test_vllm_plugin.py, tests/test_vllm_mamba2_plugin.py), run in a child process;
* (GPU) ``statequant.apply(model, fmt, schedule, backend='packed')`` drives a small fla Gated DeltaNet model through the
  sm_100a kernels (the scenario of the reference's tests/test_packed_backend.py:49-77).

Where the reference is looked for: the directory named by STATEQUANT_REF_SRC (its ``src``), else a checkout next to this
repository (``../reference/src``), else the install under ``baseline/_ref`` (baseline/install_reference.sh).  The
reference's test files are taken from STATEQUANT_REF_TESTS or ``../reference/tests``.  Tests skip when what they need is
absent.
"""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ref_src():
    for c in (os.environ.get('STATEQUANT_REF_SRC'), os.path.join(ROOT, '..', 'reference', 'src'),
              os.path.join(ROOT, 'baseline', '_ref')):
        if c and os.path.isdir(os.path.join(c, 'statequant')):
            return os.path.abspath(c)
    return None


def _ref_tests():
    for c in (os.environ.get('STATEQUANT_REF_TESTS'), os.path.join(ROOT, '..', 'reference', 'tests')):
        if c and os.path.isfile(os.path.join(c, 'test_vllm_plugin.py')):
            return os.path.abspath(c)
    return None


def _child(code, env=None, timeout=900):
    e = dict(os.environ, PYTHONDONTWRITEBYTECODE='1', **(env or {}))
    return subprocess.run([sys.executable, '-c', code], capture_output=True, text=True, env=e, timeout=timeout)


def test_bind_reference_on_the_real_package():
    src = _ref_src()
    if src is None:
        pytest.skip('no reference package found')
    code = f'''
import sys
sys.dont_write_bytecode = True
sys.path[:0] = [{src!r}, {ROOT!r}]
from statequant_b200.integrations import binding
done = binding.bind_reference()
import statequant, statequant.kernels as RK, statequant.kernels.slots as RS, statequant.kernels.mamba2 as RM
import statequant.kernels.kda as RD, statequant.kernels.fold as RF
import statequant_b200.kernels as K
for n in ('PackedGDNState', 'SlotLayout', 'PackedMamba2State', 'Mamba2SlotLayout', 'PackedKDAState', 'KDASlotLayout',
          'pack', 'unpack', 'pack_vk', 'unpack_vk', 'packed_format'):
    assert getattr(RK, n) is getattr(K, n), n
assert RS.SlotLayout is K.SlotLayout and RM.Mamba2SlotLayout is K.Mamba2SlotLayout and RD.KDASlotLayout is K.KDASlotLayout
assert RF.PackedGDNState is K.PackedGDNState
from statequant.kernels._stepquant_triton import fit
from statequant_b200.kernels.gga import fit as ours
assert fit is ours
# the reference's packed carrier resolves the class at call time: it now builds this package's state
import statequant.patch as P, inspect
assert 'PackedGDNState' in inspect.getsource(P._PackedCarry)
# layouts of the reference's own presets have the reference's byte counts
q = statequant.Quantizer
assert RK.SlotLayout(q(4, 'k', 64), 32, 16, 128, 128).nbytes == 329728
assert RK.SlotLayout(q(8, 'k', 32), 32, 16, 128, 128).nbytes == 608256
assert RK.Mamba2SlotLayout(q(8, 'k', 32), 128, 8, 128, 64).nbytes == 1195136
assert RK.KDASlotLayout(q(4, 'k', 64), 32, 128, 128).nbytes == 492672
print('BOUND', len(done))
'''
    r = _child(code)
    assert r.returncode == 0 and 'BOUND' in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_reference_calculator_tests_pass_on_rebound_layouts():
    """The reference's own plugin tests (GDN and Mamba2 state-shape / dtype calculators, layer-kind selection), run
    unmodified against vLLM with this package's layouts bound under the reference's names."""
    src, tests = _ref_src(), _ref_tests()
    if src is None or tests is None:
        pytest.skip('no reference checkout with its tests found')
    pytest.importorskip('vllm')
    code = f'''
import sys
sys.dont_write_bytecode = True
sys.path[:0] = [{src!r}, {tests!r}, {ROOT!r}]
from statequant_b200.integrations import binding
binding.bind_reference()
import pytest
sys.exit(pytest.main([{os.path.join(tests, "test_vllm_plugin.py")!r}, {os.path.join(tests, "test_vllm_mamba2_plugin.py")!r},
                      '-q', '-x', '-p', 'no:cacheprovider']))
'''
    r = _child(code, env={'STATEQUANT_VLLM_LAYERS': 'gdn,mamba2'})
    assert r.returncode == 0 and ' passed' in r.stdout and 'failed' not in r.stdout, r.stdout[-3000:] + r.stderr[-2000:]


def _greedy(model, ids, n, forced):
    """Logits of the prompt's last position and of n decode steps fed a fixed continuation."""
    with torch.no_grad():
        out = model(input_ids=ids, use_cache=True)
        logits, pkv = [out.logits[:, -1]], out.past_key_values
        for i in range(n):
            out = model(input_ids=forced[:, i:i + 1], past_key_values=pkv, use_cache=True)
            pkv = out.past_key_values
            logits.append(out.logits[:, -1])
    return torch.stack(logits, 1).float()


@pytest.mark.gpu
def test_hf_packed_backend_runs_on_these_kernels():
    """``sq.apply(model, fmt, schedule, backend='packed')`` of the real reference package, rebound, on a two-layer fla
    Gated DeltaNet (2 heads of 128): the bf16-state control tracks the unpatched model; int4 and int8 states stay as
    close to the reference's own fake-quant path as the reference's test asks (a quarter of the quantisation error);
    and the decode steps are launches of this library."""
    src = os.path.join(ROOT, 'baseline', '_ref')
    if not os.path.isdir(os.path.join(src, 'statequant')):
        pytest.skip('the reference is not installed under baseline/_ref')
    pytest.importorskip('fla')
    sys.path.insert(0, src)
    try:
        from statequant_b200 import _cabi
        from statequant_b200.integrations import binding
        binding.bind_reference()
        import statequant as rsq
        from fla.models import GatedDeltaNetConfig, GatedDeltaNetForCausalLM
        torch.manual_seed(0)
        cfg = GatedDeltaNetConfig(hidden_size=256, num_hidden_layers=2, num_heads=2, head_dim=128, expand_v=1,
                                  vocab_size=512, fuse_cross_entropy=False)
        model = GatedDeltaNetForCausalLM(cfg).cuda().to(torch.bfloat16).eval()
        g = torch.Generator().manual_seed(1)
        x = torch.randint(0, 512, (2, 256), generator=g).cuda()
        forced = torch.randint(0, 512, (2, 24), generator=g).cuda()
        rel = lambda a, b: ((a - b).norm() / b.norm()).item()                              # noqa: E731
        base = _greedy(model, x, 24, forced)
        n0 = _cabi.launch_count()
        with rsq.apply(model, rsq.FloatCast('bf16'), rsq.Schedule(prefill=256, decode=8, buffer_bits=0), backend='packed'):
            ctl = _greedy(model, x, 24, forced)
        assert _cabi.launch_count() - n0 >= 24 * 2, 'the packed decode steps did not go through this library'
        assert rel(ctl, base) < 2e-2, rel(ctl, base)
        for fmt, bb in ((rsq.Quantizer(4, 'k', 64, scale_dtype='fp16'), 16), (rsq.Quantizer(4, 'k', 64, scale_dtype='fp16'), 8),
                        (rsq.Quantizer(8, 'k', 32, scale_dtype='fp16'), 8), (rsq.Quantizer(4, 'v', 32, scale_dtype='fp16'), 16)):
            n1 = _cabi.launch_count()
            with rsq.apply(model, fmt, rsq.Schedule(prefill=256, decode=8, buffer_bits=bb), backend='packed'):
                packed = _greedy(model, x, 24, forced)
            assert _cabi.launch_count() - n1 >= 24 * 2
            with rsq.apply(model, fmt, rsq.Schedule(prefill=256, decode=8, buffer_bits=0)):
                ref = _greedy(model, x, 24, forced)
            print(f'\\n{fmt.bits}-bit {fmt.axis}{fmt.group}, buffer {bb}: packed vs reference path {rel(packed, ref):.3e}, '
                  f'reference path vs fp {rel(ref, base):.3e}')
            assert rel(packed, ref) < 0.25 * rel(ref, base) + 2e-2, (rel(packed, ref), rel(ref, base))
    finally:
        sys.path.remove(src)
