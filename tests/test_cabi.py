"""CPU-side checks of the C ABI: the library builds, loads, exports every declared symbol, and refuses bad
arguments before any launch (no compute call needs a GPU here)."""
import ctypes as C
import os
import re

import pytest
import torch

import statequant_b200 as sq
from statequant_b200 import _cabi
from statequant_b200.kernels import KDASlotLayout, Mamba2SlotLayout, SlotLayout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    hdr = open(os.path.join(ROOT, 'include', 'statequant_b200.h')).read()
    hdr = re.sub(r'/\*.*?\*/', '', hdr, flags=re.S)
    return sorted(set(re.findall(r'\b(sqb_[a-z0-9_]+)\s*\(', hdr)))


def test_library_exports_every_declared_symbol():
    L = _cabi.lib()
    names = declared_symbols()
    assert {'sqb_gdn_step', 'sqb_mamba2_step', 'sqb_kda_step', 'sqb_last_error', 'sqb_abi_version'} <= set(names)
    for n in names:
        assert hasattr(L, n), n
    assert L.sqb_abi_version() == _cabi.ABI_VERSION


def test_struct_sizes_match_header():
    """ctypes mirrors of the structs have the C compiler's size (a field added on one side only would shift it)."""
    import subprocess
    import tempfile
    src = '#include <stdio.h>\n#include "statequant_b200.h"\nint main(){printf("%zu %zu %zu %zu", sizeof(sqb_state_t), ' \
          'sizeof(sqb_gdn_inputs_t), sizeof(sqb_mamba2_inputs_t), sizeof(sqb_kda_inputs_t));return 0;}'
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, 't.c'), 'w').write(src)
        subprocess.run(['gcc', '-I', os.path.join(ROOT, 'include'), os.path.join(d, 't.c'), '-o', os.path.join(d, 't')],
                       check=True)
        sizes = [int(x) for x in subprocess.run([os.path.join(d, 't')], capture_output=True, text=True).stdout.split()]
    assert sizes == [C.sizeof(_cabi.State), C.sizeof(_cabi.GdnInputs), C.sizeof(_cabi.Mamba2Inputs),
                     C.sizeof(_cabi.KdaInputs)]


def test_bad_arguments_are_refused_with_a_message():
    L = _cabi.lib()
    st = _cabi.State()
    a = _cabi.GdnInputs()
    st.bits, st.buffer_bits, st.m, st.hv, st.hk, st.dk, st.dv, st.group, st.axis_k = 5, 8, 8, 4, 2, 128, 128, 64, 1
    assert L.sqb_gdn_step(C.byref(st), C.byref(a), None) == -1 and b'bits 5' in L.sqb_last_error()
    st.bits, st.m = 4, 6
    assert L.sqb_gdn_step(C.byref(st), C.byref(a), None) == -1 and b'power of two' in L.sqb_last_error()
    st.m, st.hk = 8, 3
    assert L.sqb_gdn_step(C.byref(st), C.byref(a), None) == -1 and b'multiple of hk' in L.sqb_last_error()
    st.hk, st.dk = 2, 80                      # rows that are not whole 16-byte chunks
    assert L.sqb_gdn_step(C.byref(st), C.byref(a), None) == -1 and b'd_k 80' in L.sqb_last_error()
    st.dk = 128
    assert L.sqb_gdn_step(C.byref(st), C.byref(a), None) == -1 and b'NULL' in L.sqb_last_error()
    assert L.sqb_gdn_step(None, C.byref(a), None) == -1
    stk = _cabi.State()
    stk.bits, stk.buffer_bits, stk.m, stk.hv, stk.hk, stk.dk, stk.dv, stk.group, stk.axis_k = 4, 8, 8, 4, 2, 128, 128, 64, 1
    assert L.sqb_kda_step(C.byref(stk), C.byref(_cabi.KdaInputs()), None) == -1 and b'KDA' in L.sqb_last_error()


def test_layout_bytes_at_baseline_shapes():
    """Exact per-slot byte counts of the serving layouts (reference: tests/test_slots.py:210-216 and the figures of
    its README: pace4 329,728, int8k 608,256, int4v 346,112, bf16 1,099,776 bytes per slot per layer)."""
    lay = SlotLayout(sq.Quantizer(4, 'k', 64), 32, 16, 128, 128, m=8, buffer_bits=8)
    b = lay.breakdown()
    assert b['S'] == 32 * 128 * 64 and b['SC'] == 32 * 128 * 2 * 2
    assert b['KB'] == 16 * 8 * 128 and b['UB'] == 32 * 8 * 128
    assert lay.nbytes == sum(-(-x // 16) * 16 for x in b.values()) == 329728
    assert list(lay.fields) == ['GB', 'GCUR', 'NPTR', 'SC', 'KBS', 'UBS', 'S', 'KB', 'UB']
    assert all(f[0] % 16 == 0 for f in lay.fields.values())
    assert SlotLayout(sq.Quantizer(8, 'k', 32), 32, 16, 128, 128).nbytes == 608256
    assert SlotLayout(sq.Quantizer(4, 'v', 32), 32, 16, 128, 128).nbytes == 346112
    assert SlotLayout('bf16', 32, 16, 128, 128).nbytes == 1099776
    assert SlotLayout('fp32', 32, 16, 128, 128).fields['S'][1] == torch.float32
    assert Mamba2SlotLayout(sq.Quantizer(8, 'k', 32), 128, 8, 128, 64).nbytes == 1195136
    k = KDASlotLayout(sq.Quantizer(4, 'k', 64), 32, 128, 128)
    assert k.nbytes == 492672 and k.fields['GB'][2] == (32, 8, 128) and k.fields['GCUR'][2] == (32, 128)
    assert SlotLayout(sq.Quantizer(4, 'k', 64), 30, 30, 96, 192).fields['SC'][2] == (30, 192, 2)   # ragged 64 + 32


def test_views_reject_misaligned_blobs():
    lay = SlotLayout(sq.Quantizer(4, 'k', 64), 4, 2, 128, 128)
    raw = torch.zeros(3, lay.nbytes + 64, dtype=torch.uint8)
    lay.views(raw[:, :lay.nbytes])
    with pytest.raises(AssertionError):
        lay.views(raw[:, 8:8 + lay.nbytes])
    with pytest.raises(AssertionError):
        lay.views(raw[:, :lay.nbytes - 16])
    with pytest.raises(AssertionError):
        lay.views(raw.to(torch.int8)[:, :lay.nbytes])


def test_unsupported_formats_raise_at_construction():
    with pytest.raises(AssertionError):
        SlotLayout(sq.Quantizer(4, 'k', 64, affine=True), 4, 2, 128, 128)
    with pytest.raises(AssertionError):
        SlotLayout(sq.Quantizer(4, 'k', 64, rotation='hadamard'), 4, 2, 128, 128)
    with pytest.raises(AssertionError):
        SlotLayout(sq.Quantizer(6, 'k', 64), 4, 2, 128, 128)
    with pytest.raises(AssertionError):
        SlotLayout(sq.Quantizer(4, 'k', 64), 4, 3, 128, 128)
    with pytest.raises(AssertionError):
        KDASlotLayout(sq.Quantizer(4, 'k', 64), 4, 96, 128)
