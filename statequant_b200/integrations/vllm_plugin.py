"""The vLLM side: what ``STATEQUANT_VLLM`` selects, the layouts the engine's state slots take, and registration.

Environment (the reference's surface, ``src/statequant/integrations/vllm_plugin.py:6-30,81-120``):

    STATEQUANT_VLLM=pace4|int4k|int4v|int8k|int8v|bf16|fp32|int<4|8><k|v>g<group>|gga:<plan.pt>[:pw]
    STATEQUANT_VLLM_M=8               decode buffer length (power of two)
    STATEQUANT_VLLM_BUFFER_BITS=8     8 (int8 + fp16 scale) or 16 (bf16)
    STATEQUANT_VLLM_LAYERS=gdn,mamba2,kda
    STATEQUANT_VLLM_PW_M=8            window length of gga:...:pw
    STATEQUANT_VLLM_FUSED, STATEQUANT_GGA_WARPS   parsed and ignored (one code path here)
    STATEQUANT_B200_FOLD=launch|inline   (this package only) where a slot's m-th token is folded: in a balanced launch
                                      of its own behind the step kernel (default under vLLM: the slots of a serving
                                      batch sit at different buffer positions, and a launch that mixes folding and
                                      plain rows ends on the long-running folding CTAs), or inside the step kernel

``register()`` is the ``vllm.general_plugins`` entry point.  The engine glue -- replacing the state-shape calculators
and the layers' ``_forward_core`` -- is Python that lives in the reference's plugin and depends on vLLM >= 0.32
internals; this module does not duplicate it.  It binds this package's layouts and kernels under the reference's
names (``binding.bind_reference``) and then lets the reference's own ``register()`` install its hooks, so every
``lay.step`` / ``lay.read`` / ``lay.write`` the engine makes lands in the sm_100a kernels.  Without the reference
package installed, ``register()`` still patches the state-shape / dtype calculators (so the memory planner sizes the
packed slots) and refuses to go further with a clear error.
"""
from __future__ import annotations

import os
import re

import torch

ENV = 'STATEQUANT_VLLM'
PRESETS = {'pace4': (4, 'k', 64), 'int4k': (4, 'k', 64), 'int4v': (4, 'v', 32), 'int8k': (8, 'k', 32),
           'int8v': (8, 'v', 32)}
LAYER_KINDS = ('gdn', 'mamba2', 'kda')
_STATE = {}


def config():
    """(fmt, m, buffer_bits, fused) from the environment, or None when the plugin is off.  ``fmt`` is a Quantizer,
    'bf16', 'fp32' or 'gga' (then ``_STATE['gga'] = (plan path, pw, window length)``)."""
    raw = os.environ.get(ENV, '').strip()
    mode = raw.lower()
    if mode in ('', '0', 'off', 'none', 'stock'):
        return None
    from ..quantizer import Quantizer
    _STATE.pop('gga', None)
    if mode.startswith('external:'):
        # An external state quantizer fn(S, layer) applied to the stored state after every fold and prefill chunk: the
        # slot then holds an UNPACKED state (fp32, or bf16 by STATEQUANT_VLLM_EXTERNAL_DTYPE) that the decode step of
        # this package advances like any other; fn itself is imported and called by the reference's forward hook
        # (vllm_plugin.py:400-410 there), on the slot layout's 'S' view.
        spec = raw[len('external:'):]
        src, _, fn = spec.rpartition(':')
        assert src and fn, f'{ENV}=external:<file.py or module>:<function>, got {spec!r}'
        fmt = os.environ.get('STATEQUANT_VLLM_EXTERNAL_DTYPE', 'fp32').strip().lower()
        assert fmt in ('fp32', 'bf16'), f'STATEQUANT_VLLM_EXTERNAL_DTYPE={fmt!r}: use fp32 or bf16'
    elif mode.startswith('gga:'):
        rest = raw[len('gga:'):]
        pw = rest.endswith(':pw')
        path = rest[:-3] if pw else rest
        assert os.path.exists(path), f'{ENV}=gga:<plan.pt>[:pw]: no plan file {path!r}'
        _STATE['gga'] = (path, pw, int(os.environ.get('STATEQUANT_VLLM_PW_M', '8')))
        fmt = 'gga'
    elif mode in ('bf16', 'fp32'):
        fmt = mode
    elif mode in PRESETS:
        fmt = Quantizer(*PRESETS[mode])
    else:
        mt = re.fullmatch(r'int([48])([kv])g(\d+)', mode)
        assert mt, (f'{ENV}={mode!r}: use pace4, int4v, int8k, int8v, bf16, fp32, gga:<plan.pt>[:pw] or '
                    f'int<4|8><k|v>g<group>')
        fmt = Quantizer(int(mt.group(1)), mt.group(2), int(mt.group(3)))
    m = int(os.environ.get('STATEQUANT_VLLM_M', '8'))
    bb = int(os.environ.get('STATEQUANT_VLLM_BUFFER_BITS', '8'))
    fz = os.environ.get('STATEQUANT_VLLM_FUSED', 'auto').strip().lower()
    assert fz in ('auto', '', '0', '1'), f'STATEQUANT_VLLM_FUSED={fz!r}: use 0, 1 or auto'
    return fmt, m, bb, (None if fz in ('auto', '') else fz == '1')


def layer_kinds():
    raw = os.environ.get('STATEQUANT_VLLM_LAYERS', '').strip().lower()
    if not raw:
        return LAYER_KINDS
    kinds = tuple(k.strip() for k in raw.split(',') if k.strip())
    assert kinds and set(kinds) <= set(LAYER_KINDS), f'STATEQUANT_VLLM_LAYERS={raw!r}: a subset of {LAYER_KINDS}'
    return kinds


def load_plan(path):
    """A STEP / GGA plan file as written by the reference's ``StepQuant.save`` (a ``torch.save`` dict holding
    ``plan`` {layer: (bits, w)} and ``group``)."""
    from ..kernels.gga import StepPlan
    d = torch.load(path, map_location='cpu', weights_only=False)
    plan = d['plan'] if isinstance(d, dict) else d.plan
    group = (d.get('group', 32) if isinstance(d, dict) else getattr(d, 'group', 32))
    return StepPlan({k: (torch.as_tensor(b), torch.as_tensor(w).float()) for k, (b, w) in plan.items()}, group,
                    name=os.path.basename(path))


def _cfg():
    if 'cfg' not in _STATE:
        _STATE['cfg'] = config()
    assert _STATE['cfg'] is not None, f'{ENV} is not set'
    return _STATE['cfg']


def layout(hv, hk, dk, dv):
    """The GDN slot layout for a layer with these per-rank head counts and dims (cached)."""
    from ..kernels import GGAPacked, SlotLayout
    fmt, m, bb, fused = _cfg()
    key = ('gdn', hv, hk, dk, dv)
    lays = _STATE.setdefault('layouts', {})
    if key not in lays:
        if fmt == 'gga':
            path, pw, pm = _STATE['gga']
            if 'gga_plan' not in _STATE:
                _STATE['gga_plan'] = load_plan(path)
            lays[key] = GGAPacked(_STATE['gga_plan'], hv, hk, dk, dv, pw=pw, m=pm)
        else:
            lays[key] = SlotLayout(fmt, hv, hk, dk, dv, m=m, buffer_bits=bb, fused=fused)
    return lays[key]


def mamba2_layout(heads, groups, d_state, head_dim):
    from ..kernels import Mamba2SlotLayout
    fmt, m, bb, _ = _cfg()
    assert fmt not in ('fp32', 'gga'), f'{ENV}={os.environ.get(ENV)!r}: GDN layers only'
    key = ('mamba2', heads, groups, d_state, head_dim)
    lays = _STATE.setdefault('layouts', {})
    if key not in lays:
        lays[key] = Mamba2SlotLayout(fmt, heads, groups, d_state, head_dim, m=m, buffer_bits=bb)
    return lays[key]


def kda_layout(heads, dk, dv):
    from ..kernels import KDASlotLayout
    fmt, m, bb, _ = _cfg()
    assert fmt not in ('fp32', 'gga'), f'{ENV}={os.environ.get(ENV)!r}: GDN layers only'
    key = ('kda', heads, dk, dv)
    lays = _STATE.setdefault('layouts', {})
    if key not in lays:
        lays[key] = KDASlotLayout(fmt, heads, dk, dv, m=m, buffer_bits=bb)
    return lays[key]


def patch_calculators():
    """vLLM's GDN state-shape / dtype calculators: the layer's second state (stock: the ssm state) becomes one uint8
    blob of ``layout.nbytes`` per slot, so the hybrid page size, the KV-cache spec and the memory planner all see the
    packed size (reference: ``vllm_plugin.py:252-279``).  Returns the original pair."""
    from vllm.model_executor.layers.mamba import mamba_utils as mu
    if 'calculators' in _STATE:
        return _STATE['calculators']
    shape0 = mu.MambaStateShapeCalculator.gated_delta_net_state_shape
    dtype0 = mu.MambaStateDtypeCalculator.gated_delta_net_state_dtype
    _STATE['calculators'] = (shape0, dtype0)

    def gated_delta_net_state_shape(cls, tp_world_size, num_k_heads, num_v_heads, head_k_dim, head_v_dim,
                                    conv_kernel_size, num_spec=0):
        assert num_spec == 0, 'statequant vLLM plugin: speculative decoding is not supported'
        conv_shape, _ = shape0(tp_world_size, num_k_heads, num_v_heads, head_k_dim, head_v_dim, conv_kernel_size,
                               num_spec)
        lay = layout(num_v_heads // tp_world_size, num_k_heads // tp_world_size, head_k_dim, head_v_dim)
        return conv_shape, (lay.nbytes,)

    def gated_delta_net_state_dtype(cls, model_dtype, mamba_cache_dtype, *a, **kw):
        conv_dtype, _ = dtype0(model_dtype, mamba_cache_dtype, *a, **kw)
        return conv_dtype, torch.uint8

    mu.MambaStateShapeCalculator.gated_delta_net_state_shape = classmethod(gated_delta_net_state_shape)
    mu.MambaStateDtypeCalculator.gated_delta_net_state_dtype = classmethod(gated_delta_net_state_dtype)
    return shape0, dtype0


def unpatch_calculators():
    from vllm.model_executor.layers.mamba import mamba_utils as mu
    if 'calculators' in _STATE:
        shape0, dtype0 = _STATE.pop('calculators')
        mu.MambaStateShapeCalculator.gated_delta_net_state_shape = shape0
        mu.MambaStateDtypeCalculator.gated_delta_net_state_dtype = dtype0


def fold_policy():
    """'launch' or 'inline' from STATEQUANT_B200_FOLD (default 'launch': continuous batching)."""
    pol = os.environ.get('STATEQUANT_B200_FOLD', 'launch').strip().lower()
    assert pol in ('launch', 'inline'), f'STATEQUANT_B200_FOLD={pol!r}: use launch or inline'
    return pol


def apply_fold_policy():
    """Select the device code path of the decode steps for this process: kernel_path 3 (step kernel that only appends +
    the fold launch) for 'launch', 0 (the fold inside the step kernel wherever the shape allows) for 'inline'."""
    from .. import _cabi
    _cabi.set_option('kernel_path', 3 if fold_policy() == 'launch' else 0)


def register():
    """``vllm.general_plugins`` entry point.  Idempotent; a no-op unless STATEQUANT_VLLM is set."""
    cfg = config()
    if cfg is None or _STATE.get('registered'):
        return
    _STATE['cfg'] = cfg
    try:
        from . import binding
        binding.bind_reference()
        from statequant.integrations import vllm_plugin as ref_plugin
    except ImportError as err:
        # The layer forward hooks are the reference package's own Python (statequant.integrations.vllm_plugin); without
        # it nothing of vLLM is touched: no calculator is patched, the engine runs its stock state.
        import warnings
        warnings.warn('statequant_b200: STATEQUANT_VLLM is set but the statequant package, whose vLLM layer hooks run '
                      f'on these kernels, cannot be imported ({err}); vLLM is left unchanged', RuntimeWarning, stacklevel=2)
        _STATE['registered'] = 'skipped'
        return
    ref_plugin.register()
    apply_fold_policy()
    _STATE['registered'] = True
