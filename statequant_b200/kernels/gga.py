"""Packed GGA / STEP mixed-bit state with the pure-write window (PW-S m) on Gated DeltaNet layers.

``GGAPacked`` mirrors the reference class of that name (``src/statequant/integrations/vllm_gga.py:182-318``): the
per-layer offset tables of a plan (per-head widths 2 / 4 / 6 / 8 bits or 16 = fp16 pivot), the slot byte layout
(``src/statequant/kernels/_gga_triton.py:3-13``), and ``step`` / ``stored`` / ``window`` / ``read`` / ``write`` /
``bits_per_value``.  The device work goes through ``sqb_gga_step`` / ``sqb_gga_store`` / ``sqb_gga_load``;
``fit`` is STEP's dual-axis fit as a stand-alone pass (``sqb_stepquant_fit``).

A plan is any object with ``plan`` ({layer: (bits [HV], w [HV, d_k])}), ``group`` (32) and ``name`` -- the reference's
``StepQuant`` / ``GGA`` methods after calibration, or ``StepPlan`` here.
"""
from __future__ import annotations

import ctypes as C
import dataclasses

import torch

from .. import _cabi
from .layout import ALIGN


@dataclasses.dataclass
class StepPlan:
    """A calibrated STEP / GGA allocation: per layer the head widths and the impact factors."""
    plan: dict
    group: int = 32
    name: str = 'gga'


def head_bytes(b, dk, dv, group=32):
    """Stored bytes of one head at width b: codes + row factors (2 bit: per 32-column group) + column factors."""
    if b == 16:
        return 2 * dk * dv
    if b == 2:
        return dk * dv // 4 + 2 * dk * (dv // group) + 2 * dv
    return dk * dv * b // 8 + 2 * dk + 2 * dv


def _al(n):
    return -(-n // ALIGN) * ALIGN


class GgaLayoutStruct(C.Structure):
    """``sqb_gga_layout_t``"""
    _fields_ = [('blob', C.c_void_p), ('stride', C.c_int64), ('offs', C.c_void_p), ('bits', C.c_void_p),
                ('w', C.c_void_p), ('qoff', C.c_int64), ('qsz', C.c_int32), ('hv', C.c_int32), ('hk', C.c_int32),
                ('dk', C.c_int32), ('dv', C.c_int32), ('m', C.c_int32), ('pw', C.c_int32), ('group', C.c_int32),
                ('reserved', C.c_int32)]


def fit(x, bits, w, group=32, has_two=None):
    """STEP's dual-axis fit of x [B, H, d_k, d_v] (fp32, CUDA) with widths bits [H] (int32, device) and impact
    factors w [H, d_k] (fp32, device): the fake-quant reconstruction (reference: ``_stepquant_triton.fit``)."""
    B, H, DK, DV = x.shape
    x = x.float().contiguous()
    y = torch.empty_like(x)
    bits = bits.to(torch.int32).contiguous()
    w = w.float().contiguous()
    L = _cabi.lib()
    _cabi.check(L.sqb_stepquant_fit(C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), C.c_void_p(bits.data_ptr()),
                                    C.c_void_p(w.data_ptr()), C.c_int64(B), H, DK, DV, group,
                                    _cabi.current_stream(x.device)), 'sqb_stepquant_fit')
    return y


class GGAPacked:
    """The packed slot for every GDN layer of a plan.  The per-head widths differ between layers, so each layer has
    its own offset table; an engine sizes one slot for all layers, so ``nbytes`` is the largest layer's."""
    per_layer = True

    def __init__(self, method, hv, hk, dk, dv, pw=False, m=8):
        assert dk & (dk - 1) == 0 and dv & (dv - 1) == 0 and dv % 32 == 0, (dk, dv)
        self.method, self.HV, self.HK, self.DK, self.DV = method, hv, hk, dk, dv
        self.pw, self.m, self.gqa = pw, m, hv // hk
        self.tables, self.bytes_per_layer = {}, {}
        for layer, (b, w) in method.plan.items():
            b = [int(x) for x in b]
            assert len(b) == hv and set(b) <= {2, 4, 6, 8, 16}, b
            offs, off = [], 16                                  # the counters come first
            for x in b:
                offs.append(off)
                off += _al(head_bytes(x, dk, dv, method.group))
            self.tables[layer] = (offs, b, w)
            self.bytes_per_layer[layer] = off
        self.QOFF = _al(max(self.bytes_per_layer.values()))
        self.QSZ = m * (dk + dv + 8)
        self.nbytes = self.QOFF + (hv * self.QSZ if pw else 0)
        self._dev = {}
        if torch.cuda.is_available():       # stage the plans now: a copy inside a CUDA-graph capture would fail
            self.prepare(torch.device('cuda', torch.cuda.current_device()))

    def __repr__(self):
        return (f'GGAPacked({self.method.name}{"+PW-S%d" % self.m if self.pw else ""}, hv={self.HV}, hk={self.HK}, '
                f'dk={self.DK}, dv={self.DV}, {self.nbytes} B/slot = max over layers; mean '
                f'{self.bits_per_value():.3f} b/value)')

    def bits_per_value(self):
        """Mean stored bits per state value over the layers (without the 16-byte counters), window included."""
        n = self.HV * self.DK * self.DV
        st = sum(sum(head_bytes(x, self.DK, self.DV, self.method.group) for x in t[1]) for t in self.tables.values())
        q = self.HV * self.QSZ * len(self.tables) if self.pw else 0
        return 8 * (st + q) / (n * len(self.tables))

    def _plan(self, layer, dev):
        key = (layer, str(dev))
        if key not in self._dev:
            offs, b, w = self.tables[layer]
            self._dev[key] = (torch.tensor(offs, dtype=torch.int32, device=dev),
                              torch.tensor(b, dtype=torch.int32, device=dev),
                              w.to(dev, torch.float32).contiguous())
        return self._dev[key]

    def prepare(self, device):
        """Move every layer's plan to the device now (so that nothing is copied during graph capture)."""
        for layer in self.tables:
            self._plan(layer, device)

    def views(self, blob):
        assert blob.dtype == torch.uint8 and blob.dim() == 2 and blob.shape[1] >= self.nbytes
        assert blob.stride(1) == 1 and blob.stride(0) % ALIGN == 0 and blob.data_ptr() % ALIGN == 0
        return {'blob': blob}

    def alloc(self, num_slots, device='cuda'):
        return torch.zeros(num_slots, self.nbytes, dtype=torch.uint8, device=device)

    def _struct(self, views, layer):
        blob = views['blob']
        offs, bits, w = self._plan(layer, blob.device)
        st = GgaLayoutStruct()
        st.blob, st.stride = blob.data_ptr(), blob.stride(0)
        st.offs, st.bits, st.w = offs.data_ptr(), bits.data_ptr(), w.data_ptr()
        st.qoff, st.qsz = self.QOFF, self.QSZ
        st.hv, st.hk, st.dk, st.dv, st.m, st.pw, st.group = self.HV, self.HK, self.DK, self.DV, self.m, int(self.pw), \
            self.method.group
        return st

    def step(self, views, idx, q, k, v, out, scale, *, g=None, beta=None, gate=None, layer=None, fused=None):
        """One decode token for every batch row on slot ``idx[b]`` (<= 0: padding row, output zeroed).  Takes the
        gate inputs ``gate=(a, b, A_log, dt_bias)``; two launches (step, window counters)."""
        from .slots import _gdn_inputs
        assert gate is not None, 'GGAPacked.step takes the gate inputs (a, b, A_log, dt_bias)'
        B = idx.shape[0]
        if B == 0:
            return out
        assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1 and v.stride(1) == self.DV
        assert q.stride(-2) == self.DK and k.stride(-2) == self.DK
        assert out.is_contiguous() and idx.dtype == torch.int32 and idx.is_contiguous()
        a = _gdn_inputs(idx, q, k, v, out[:B], scale, None, None, gate, True)
        st = self._struct(views, layer)
        _cabi.check(_cabi.lib().sqb_gga_step(C.byref(st), C.byref(a), _cabi.current_stream(q.device)), 'sqb_gga_step')
        return out

    @torch.no_grad()
    def stored(self, views, idx, layer):
        """The stored states of slots idx, canonical fp32 [P, HV, d_k, d_v] (without the window)."""
        idx32 = idx.to(torch.int32).contiguous()
        P = idx32.shape[0]
        Y = torch.empty(P, self.HV, self.DK, self.DV, device=idx.device)
        if P:
            st = self._struct(views, layer)
            _cabi.check(_cabi.lib().sqb_gga_load(C.byref(st), C.c_void_p(idx32.data_ptr()), C.c_int64(P),
                                                 C.c_void_p(Y.data_ptr()), _cabi.current_stream(idx.device)),
                        'sqb_gga_load')
        return Y

    @torch.no_grad()
    def window(self, views, idx):
        """The queued pairs of slots idx as reconstructed fp32 (P [n, m, HV, d_k], V [n, m, HV, d_v]) in ring order
        from the oldest, and the counts; dead entries zeroed (torch; reference: ``vllm_gga.py:275-293``)."""
        li = idx.long()
        blob = views['blob'][li]
        m, HV, DK, DV = self.m, self.HV, self.DK, self.DV
        ct = blob[:, :16].view(torch.int32)
        n, hd = ct[:, 0], ct[:, 1]
        Qb = blob[:, self.QOFF:self.QOFF + HV * self.QSZ].reshape(-1, HV, self.QSZ)
        Pc = Qb[..., :m * DK].contiguous().view(torch.float8_e4m3fn).float().view(-1, HV, m, DK)
        Vc = Qb[..., m * DK:m * (DK + DV)].contiguous().view(torch.float8_e4m3fn).float().view(-1, HV, m, DV)
        sc = Qb[..., m * (DK + DV):].contiguous().view(torch.float32).view(-1, HV, 2, m)
        Pf, Vf = Pc * sc[:, :, 0, :, None], Vc * sc[:, :, 1, :, None]
        order = (hd[:, None] + torch.arange(m, device=li.device)[None, :]) % m
        Pf = torch.gather(Pf, 2, order[:, None, :, None].expand(-1, HV, -1, DK)).transpose(1, 2)
        Vf = torch.gather(Vf, 2, order[:, None, :, None].expand(-1, HV, -1, DV)).transpose(1, 2)
        live = (torch.arange(m, device=li.device)[None, :] < n[:, None])[:, :, None, None]
        return torch.where(live, Pf, 0.), torch.where(live, Vf, 0.), n

    @torch.no_grad()
    def read(self, views, idx, layer=None):
        """Logical state (stored + window), value-major fp32 [P, HV, d_v, d_k]."""
        S = self.stored(views, idx, layer)
        if self.pw and idx.shape[0]:
            P, V, _ = self.window(views, idx)
            _, bits, _ = self._plan(layer, idx.device)
            nonp = (bits != 16)[None, :, None, None].float()
            S = S + torch.einsum('bmhk,bmhv->bhkv', P, V) * nonp
        return S.transpose(-1, -2)

    @torch.no_grad()
    def write(self, views, idx, S, layer=None):
        """Fit + pack value-major states S [P, HV, d_v, d_k] into slots idx; empty the window."""
        idx32 = idx.to(torch.int32).contiguous()
        P = idx32.shape[0]
        if P == 0:
            return
        X = S.float().transpose(-1, -2).contiguous()
        st = self._struct(views, layer)
        _cabi.check(_cabi.lib().sqb_gga_store(C.byref(st), C.c_void_p(idx32.data_ptr()), C.c_int64(P),
                                              C.c_void_p(X.data_ptr()), _cabi.current_stream(S.device)),
                    'sqb_gga_store')
