"""Drop the sm_100a kernels into an installed ``statequant`` (the reference package) without touching its files.

    import statequant_b200.integrations.binding as b
    b.bind_reference()
    with statequant.apply(model, statequant.pace4(paper=False), backend='packed'): ...

After ``bind_reference()`` the names the reference's hosts resolve at call time -- ``statequant.kernels.PackedGDNState``
(used by ``patch._PackedCarry``, ``src/statequant/patch.py:195``), ``SlotLayout`` / ``Mamba2SlotLayout`` /
``KDASlotLayout`` (used by the vLLM plugin, ``integrations/vllm_plugin.py:123-141``, ``vllm_mamba2.py``,
``vllm_kda.py``), ``integrations.vllm_gga.GGAPacked`` and ``kernels._stepquant_triton.fit`` -- are this package's
classes, which keep the reference's constructor and method signatures and its byte layout.  Everything else of the
reference (HF patching, vLLM forward hooks, calibration) keeps running its own Python.
"""
from __future__ import annotations

import importlib
import sys
import types

from .. import kernels as K
from ..kernels import gga as G

_BOUND = {}

_NAMES = ['PackedGDNState', 'SlotLayout', 'PackedMamba2State', 'Mamba2SlotLayout', 'PackedKDAState', 'KDASlotLayout',
          'pack', 'unpack', 'pack_vk', 'unpack_vk', 'packed_format']


def _triton_stub():
    """The reference imports triton lazily inside its launch paths only; its module ``_stepquant_triton`` imports it
    at module level, so ``fit`` is bound through a stand-in module when Triton is not wanted."""
    m = types.ModuleType('statequant.kernels._stepquant_triton')
    m.fit = G.fit
    return m


def bind_reference(package='statequant'):
    """Replace the packed-path classes of the installed reference package by this package's.  Idempotent.
    Returns the list of (module, attribute) pairs that were rebound."""
    if _BOUND.get(package):
        return _BOUND[package]
    ref = importlib.import_module(package)
    done = []

    def put(modname, attr, obj):
        mod = importlib.import_module(modname)
        setattr(mod, attr, obj)
        done.append((modname, attr))

    for n in _NAMES:
        put(f'{package}.kernels', n, getattr(K, n))
    put(f'{package}.kernels.fold', 'PackedGDNState', K.PackedGDNState)
    put(f'{package}.kernels.slots', 'SlotLayout', K.SlotLayout)
    put(f'{package}.kernels.mamba2', 'PackedMamba2State', K.PackedMamba2State)
    put(f'{package}.kernels.mamba2', 'Mamba2SlotLayout', K.Mamba2SlotLayout)
    put(f'{package}.kernels.kda', 'PackedKDAState', K.PackedKDAState)
    put(f'{package}.kernels.kda', 'KDASlotLayout', K.KDASlotLayout)
    # the STEP fit: GGALayout._quant and StepQuant.quantize import it at call time
    sys.modules[f'{package}.kernels._stepquant_triton'] = _triton_stub()
    done.append((f'{package}.kernels._stepquant_triton', 'fit'))
    try:
        put(f'{package}.integrations.vllm_gga', 'GGAPacked', K.GGAPacked)
    except Exception:                      # the integrations subpackage needs nothing else of vLLM to import
        pass
    _BOUND[package] = done
    ref._statequant_b200_bound = True
    return done


def bind_conv_update(module, name='causal_conv1d_update'):
    """Route the plain decode case of ``module.<name>`` -- the vLLM model module's ``causal_conv1d_update``, which the
    reference's forward calls right before the packed step (``integrations/vllm_plugin.py:379-381``) -- to this
    package's kernel.  Calls the kernel does not take (speculative decoding, varlen batches, prefix-cache block
    indices, host tensors) go to the original.  Idempotent; returns the original function."""
    from ..kernels.conv import causal_conv1d_update as ours
    orig = getattr(module, name)
    if getattr(orig, '_statequant_b200', False):
        return orig._original

    def causal_conv1d_update(x, conv_state, weight, bias=None, activation=None, conv_state_indices=None, **kw):
        plain = (x.is_cuda and x.dim() == 2 and 2 <= weight.size(1) <= 4
                 and all(kw.get(k) is None for k in ('num_accepted_tokens', 'query_start_loc',
                                                     'block_idx_last_scheduled_token', 'initial_state_idx')))
        if not plain:
            return orig(x, conv_state, weight, bias, activation, conv_state_indices=conv_state_indices, **kw)
        return ours(x, conv_state, weight, bias, activation, conv_state_indices,
                    null_block_id=kw.get('null_block_id', 0))

    causal_conv1d_update._statequant_b200 = True
    causal_conv1d_update._original = orig
    setattr(module, name, causal_conv1d_update)
    return orig
