"""Packed (real-storage) decode path on B200: int4 / int8 / bf16 recurrent state with a delta-value decode buffer.

Same names as the reference's ``statequant.kernels`` (``src/statequant/kernels/__init__.py:10-18``); the
``Reference*State`` torch classes of the reference are test oracles there and are not part of this package.
"""
from .formats import pack, pack_vk, packed_format, unpack, unpack_vk
from .fold import PackedGDNState
from .slots import SlotLayout
from .mamba2 import Mamba2SlotLayout, PackedMamba2State, mamba2_recurrence
from .kda import KDASlotLayout, PackedKDAState, kda_recurrence
from .gga import GGAPacked, StepPlan, head_bytes
from .conv import causal_conv1d_update, split_qkv

__all__ = ['PackedGDNState', 'SlotLayout', 'pack', 'unpack', 'pack_vk', 'unpack_vk', 'packed_format',
           'PackedMamba2State', 'Mamba2SlotLayout', 'mamba2_recurrence',
           'PackedKDAState', 'KDASlotLayout', 'kda_recurrence', 'GGAPacked', 'StepPlan', 'head_bytes',
           'causal_conv1d_update', 'split_qkv']
