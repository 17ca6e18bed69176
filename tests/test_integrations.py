"""Host-side bindings (CPU): the STATEQUANT_VLLM surface, the slot sizes handed to vLLM's memory planner, and the
rebinding of an installed reference package onto this package's classes."""
import os

import pytest
import torch

import statequant_b200 as sq
from statequant_b200.integrations import vllm_plugin as P
from statequant_b200.kernels import GGAPacked, KDASlotLayout, Mamba2SlotLayout, SlotLayout


@pytest.fixture
def env(monkeypatch):
    def set_(**kw):
        for k in list(os.environ):
            if k.startswith('STATEQUANT_'):
                monkeypatch.delenv(k)
        for k, v in kw.items():
            monkeypatch.setenv(k, v)
        P._STATE.clear()
    yield set_
    P._STATE.clear()


def test_config_parsing(env):
    env()
    assert P.config() is None
    env(STATEQUANT_VLLM='pace4')
    fmt, m, bb, fused = P.config()
    assert (fmt.bits, fmt.axis, fmt.group, m, bb, fused) == (4, 'k', 64, 8, 8, None)
    env(STATEQUANT_VLLM='int8vg64', STATEQUANT_VLLM_M='4', STATEQUANT_VLLM_BUFFER_BITS='16', STATEQUANT_VLLM_FUSED='1')
    fmt, m, bb, fused = P.config()
    assert (fmt.bits, fmt.axis, fmt.group, m, bb, fused) == (8, 'v', 64, 4, 16, True)
    env(STATEQUANT_VLLM='bf16')
    assert P.config()[0] == 'bf16'
    env(STATEQUANT_VLLM='int5k')
    with pytest.raises(AssertionError):
        P.config()
    env(STATEQUANT_VLLM='pace4', STATEQUANT_VLLM_LAYERS='gdn,mamba2')
    assert P.layer_kinds() == ('gdn', 'mamba2')
    env(STATEQUANT_VLLM='pace4', STATEQUANT_VLLM_LAYERS='rwkv')
    with pytest.raises(AssertionError):
        P.layer_kinds()


def test_layout_factories(env, tmp_path):
    env(STATEQUANT_VLLM='pace4')
    lay = P.layout(32, 16, 128, 128)
    assert isinstance(lay, SlotLayout) and lay.nbytes == 329728 and P.layout(32, 16, 128, 128) is lay
    assert isinstance(P.mamba2_layout(128, 8, 128, 64), Mamba2SlotLayout)
    assert isinstance(P.kda_layout(32, 128, 128), KDASlotLayout)
    plan = {'plan': {l: (torch.tensor([[4, 6, 4, 4, 6, 4][l % 6]] * 32), torch.ones(32, 128)) for l in range(24)},
            'group': 32}
    path = str(tmp_path / 'plan.pt')
    torch.save(plan, path)
    env(STATEQUANT_VLLM=f'gga:{path}:pw')
    lay = P.layout(32, 16, 128, 128)
    assert isinstance(lay, GGAPacked) and lay.pw and lay.nbytes == 477200


def test_vllm_calculators_see_packed_slot_size(env):
    """vLLM's own calculators, patched, hand the packed slot size to the memory planner (reference:
    tests/test_vllm_plugin.py)."""
    mu = pytest.importorskip('vllm.model_executor.layers.mamba.mamba_utils')
    if not hasattr(mu.MambaStateShapeCalculator, 'gated_delta_net_state_shape'):
        pytest.skip('this vLLM has no GDN state calculators')
    env(STATEQUANT_VLLM='int8k')
    shape0, dtype0 = P.patch_calculators()
    try:
        conv, ssm = mu.MambaStateShapeCalculator.gated_delta_net_state_shape(1, 16, 32, 128, 128, 4)
        assert ssm == (608256,)
        assert conv == shape0(1, 16, 32, 128, 128, 4)[0]
        conv2, ssm2 = mu.MambaStateShapeCalculator.gated_delta_net_state_shape(2, 16, 32, 128, 128, 4)
        assert ssm2 == (SlotLayout(sq.Quantizer(8, 'k', 32), 16, 8, 128, 128).nbytes,)
        dts = mu.MambaStateDtypeCalculator.gated_delta_net_state_dtype(torch.bfloat16, 'auto')
        assert dts[1] == torch.uint8
    finally:
        P.unpatch_calculators()
    assert mu.MambaStateShapeCalculator.gated_delta_net_state_shape(1, 16, 32, 128, 128, 4)[1] != (608256,)


def test_bind_reference_rebinds_a_package(tmp_path, monkeypatch):
    """A stand-in package with the reference's module layout is rebound onto this package's classes."""
    root = tmp_path / 'fakeref'
    for d in ('', 'kernels', 'integrations'):
        (root / d).mkdir(parents=True, exist_ok=True)
        (root / d / '__init__.py').write_text('')
    for m in ('fold', 'slots', 'mamba2', 'kda'):
        (root / 'kernels' / f'{m}.py').write_text('PackedGDNState = SlotLayout = None\n')
    (root / 'integrations' / 'vllm_gga.py').write_text('GGAPacked = None\n')
    monkeypatch.syspath_prepend(str(tmp_path))
    from statequant_b200.integrations import binding
    done = binding.bind_reference('fakeref')
    import fakeref.kernels as FK
    import fakeref.kernels.slots as FS
    import fakeref.integrations.vllm_gga as FG
    from fakeref.kernels._stepquant_triton import fit
    from statequant_b200.kernels.gga import fit as our_fit
    assert FK.PackedGDNState is sq.kernels.PackedGDNState and FS.SlotLayout is SlotLayout
    assert FG.GGAPacked is GGAPacked and fit is our_fit
    assert ('fakeref.kernels', 'pack_vk') in done and binding.bind_reference('fakeref') is done


def test_register_without_the_reference_package_leaves_vllm_alone():
    """STATEQUANT_VLLM set, `statequant` not importable: a warning, no calculator patched, no exception."""
    import subprocess
    import sys
    code = (
        "import sys, warnings\n"
        "sys.modules['statequant'] = None\n"                      # import statequant -> ImportError
        "from statequant_b200.integrations import vllm_plugin as p\n"
        "with warnings.catch_warnings(record=True) as w:\n"
        "    warnings.simplefilter('always')\n"
        "    p.register()\n"
        "assert any('left unchanged' in str(x.message) for x in w), [str(x.message) for x in w]\n"
        "assert p._STATE.get('registered') == 'skipped'\n"
        "p.register()\n"                                          # idempotent
        "print('ok')\n")
    env = dict(os.environ, STATEQUANT_VLLM='pace4')
    env.pop('STATEQUANT_REF_SRC', None)
    r = subprocess.run([sys.executable, '-c', code], capture_output=True, text=True, env=env,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and 'ok' in r.stdout, r.stdout + r.stderr


def test_external_quantizer_mode_is_an_unpacked_slot(monkeypatch):
    """STATEQUANT_VLLM=external:<src>:<fn>: the reference's forward hook applies fn to the stored state; here the mode
    means an fp32 (or bf16) slot, whose 'S' view is the [slots, HV, d_v, d_k] tensor that hook reads and writes."""
    monkeypatch.setenv('STATEQUANT_VLLM', 'external:my_pkg.quant:fake_quant')
    fmt, m, bb, fused = P.config()
    assert (fmt, m, bb, fused) == ('fp32', 8, 8, None)
    monkeypatch.setenv('STATEQUANT_VLLM_EXTERNAL_DTYPE', 'bf16')
    assert P.config()[0] == 'bf16'
    monkeypatch.setenv('STATEQUANT_VLLM', 'external:nofunction')
    with pytest.raises(AssertionError):
        P.config()
    lay = SlotLayout('fp32', 4, 2, 128, 128, m=8)
    views = lay.views(torch.zeros(3, lay.nbytes, dtype=torch.uint8))
    assert views['S'].dtype == torch.float32 and tuple(views['S'].shape) == (3, 4, 128, 128)
    views['S'][torch.tensor([1])] = 0.5                       # what the hook does: an indexed write through the view
    assert float(lay.read(views, torch.tensor([1], dtype=torch.int32)).mean()) == 0.5


def test_bind_conv_update_routes_only_the_plain_decode_case():
    """Host tensors, speculative decoding and varlen calls keep going to the module's own function."""
    import types
    from statequant_b200.integrations import binding
    calls = []

    def original(x, conv_state, weight, bias=None, activation=None, conv_state_indices=None, **kw):
        calls.append(sorted(kw))
        return x

    mod = types.SimpleNamespace(causal_conv1d_update=original)
    assert binding.bind_conv_update(mod) is original
    assert binding.bind_conv_update(mod) is original                  # idempotent
    x, st, w = torch.zeros(2, 8), torch.zeros(3, 8, 3), torch.zeros(8, 4)
    assert mod.causal_conv1d_update(x, st, w) is x                    # host tensors
    assert mod.causal_conv1d_update(x, st, w, num_accepted_tokens=torch.ones(2)) is x
    assert calls == [[], ['num_accepted_tokens']]


def test_fold_policy_env(monkeypatch):
    from statequant_b200.integrations import vllm_plugin as vp
    monkeypatch.delenv('STATEQUANT_B200_FOLD', raising=False)
    assert vp.fold_policy() == 'launch'
    monkeypatch.setenv('STATEQUANT_B200_FOLD', 'inline')
    assert vp.fold_policy() == 'inline'
    monkeypatch.setenv('STATEQUANT_B200_FOLD', 'sometimes')
    with pytest.raises(AssertionError):
        vp.fold_policy()
