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
import itertools

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
    """Stored bytes of one head at width b.  A packed head is its d_k x d_v codes, one fp16 column factor per value
    channel, and fp16 row factors: one per key row, except at 2 bits where every ``group`` columns of a row have
    their own.  Width 16 is the fp16 pivot: the values themselves, no factors."""
    cells = dk * dv
    if b == 16:
        return 2 * cells
    row_factors = dk * (dv // group if b == 2 else 1)
    return cells * b // 8 + 2 * (row_factors + dv)


def _al(n):
    return -(-n // ALIGN) * ALIGN


class GgaLayoutStruct(C.Structure):
    """``sqb_gga_layout_t``"""
    _fields_ = [('blob', C.c_void_p), ('stride', C.c_int64), ('offs', C.c_void_p), ('bits', C.c_void_p),
                ('w', C.c_void_p), ('qoff', C.c_int64), ('qsz', C.c_int32), ('hv', C.c_int32), ('hk', C.c_int32),
                ('dk', C.c_int32), ('dv', C.c_int32), ('m', C.c_int32), ('pw', C.c_int32), ('group', C.c_int32),
                ('flags', C.c_int32)]


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

    WIDTHS = (2, 4, 6, 8, 16)
    COUNTERS = 16                   # bytes in front of the first head: (count, ring head) of the window, padding

    def __init__(self, method, hv, hk, dk, dv, pw=False, m=8):
        for d in (dk, dv):
            assert d > 0 and d & (d - 1) == 0, f'head dims are powers of two, got {dk} x {dv}'
        assert dv % 32 == 0 and hv % hk == 0, (dv, hv, hk)
        self.method, self.pw, self.m = method, pw, m
        self.HV, self.HK, self.DK, self.DV, self.gqa = hv, hk, dk, dv, hv // hk
        # per layer: every head's byte offset in the slot (heads back to back, each padded to the alignment), its
        # width, the impact factors; ``tables`` / ``bytes_per_layer`` are the reference's names for them
        self.tables, self.bytes_per_layer = {}, {}
        for layer, (widths, impact) in method.plan.items():
            widths = [int(x) for x in widths]
            assert len(widths) == hv and all(x in self.WIDTHS for x in widths), widths
            sizes = [_al(head_bytes(x, dk, dv, method.group)) for x in widths]
            ends = list(itertools.accumulate(sizes, initial=self.COUNTERS))
            self.tables[layer] = (ends[:-1], widths, impact)
            self.bytes_per_layer[layer] = ends[-1]
        # the window queue (per head: m key rows + m value rows of e4m3, 2 m fp32 scales) follows the largest layer
        self.QOFF = _al(max(self.bytes_per_layer.values()))
        self.QSZ = m * (dk + dv) + 2 * m * 4
        self.nbytes = self.QOFF + (hv * self.QSZ if pw else 0)
        self._dev = {}
        if torch.cuda.is_available():       # stage the plans now: a copy inside a CUDA-graph capture would fail
            self.prepare(torch.device('cuda', torch.cuda.current_device()))

    def __repr__(self):
        widths = sorted({x for t in self.tables.values() for x in t[1]})
        win = f' + window of {self.m}' if self.pw else ''
        return (f'<GGAPacked {self.method.name}{win} | widths {widths} over {len(self.tables)} layers, '
                f'{self.bits_per_value():.2f} bits per value | hv={self.HV}, hk={self.HK}, dk={self.DK}, dv={self.DV} | '
                f'{self.nbytes} B per slot>')

    def bits_per_value(self):
        """Mean stored bits per state value over the layers (without the 16-byte counters), window included."""
        per_layer = [sum(head_bytes(x, self.DK, self.DV, self.method.group) for x in widths) +
                     (self.HV * self.QSZ if self.pw else 0) for _, widths, _ in self.tables.values()]
        return 8. * sum(per_layer) / (len(per_layer) * self.HV * self.DK * self.DV)

    def _plan(self, layer, dev):
        """(offsets int32 [HV], widths int32 [HV], impact factors fp32 [HV, d_k]) of a layer on device ``dev``."""
        have = self._dev.get((layer, str(dev)))
        if have is None:
            offsets, widths, impact = self.tables[layer]
            have = tuple(torch.tensor(x, dtype=torch.int32, device=dev) for x in (offsets, widths)) + \
                (impact.to(device=dev, dtype=torch.float32).contiguous(),)
            self._dev[(layer, str(dev))] = have
        return have

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
        st.flags = int(all(x in (4, 6, 8) for x in self.tables[layer][1]))         # SQB_GGA_ALL_PACKED
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
        from the oldest, and the counts; dead entries zeroed (torch; reference: ``vllm_gga.py:275-293``).

        A head's queue record is, in this order: m key rows and m value rows of e4m3 codes, then m fp32 key scales
        and m fp32 value scales; the slot's first 16 bytes hold (count, head of the ring) as int32."""
        rows = views['blob'][idx.long()]
        m, HV, DK, DV = self.m, self.HV, self.DK, self.DV
        count, head = rows[:, :8].view(torch.int32).unbind(1)
        rec = rows[:, self.QOFF:self.QOFF + HV * self.QSZ].unflatten(1, (HV, self.QSZ))
        kc, vc, ks, vs = rec.split([m * DK, m * DV, 4 * m, 4 * m], dim=-1)

        def entries(codes, scales, d):          # -> [n, m (ring position), HV, d]
            x = codes.contiguous().view(torch.float8_e4m3fn).float().unflatten(-1, (m, d))
            return (x * scales.contiguous().view(torch.float32)[..., None]).transpose(1, 2)

        age = torch.arange(m, device=rows.device)
        ring = (head[:, None] + age) % m                                  # position of the j-th oldest entry
        live = (age < count[:, None])[..., None, None]
        who = torch.arange(rows.shape[0], device=rows.device)[:, None]
        P, V = entries(kc, ks, DK)[who, ring], entries(vc, vs, DV)[who, ring]
        return P.where(live, 0.), V.where(live, 0.), count        # not a product: a dead entry may decode to NaN

    @torch.no_grad()
    def read(self, views, idx, layer=None):
        """Logical state (stored + window), value-major fp32 [P, HV, d_v, d_k].  The window adds the outer products
        of its live pairs to every packed head; a pivot head (width 16) takes its writes at once and has none
        pending."""
        S = self.stored(views, idx, layer)
        if self.pw and idx.numel():
            keys, values, _ = self.window(views, idx)
            packed = self._plan(layer, idx.device)[1] != 16
            S[:, packed] += torch.einsum('bmhk,bmhv->bhkv', keys, values)[:, packed]
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
