"""Memory safety of the kernels without a sanitizer: every output tensor is carved out of a larger buffer whose
guard regions hold a sentinel, the entry points are called through the C ABI, and the guards must come back
untouched.  Shapes cover the TMA path (clipped tiles in time and channels) and the bounds-checked plain path."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
GUARD = 4096          # elements on either side; a multiple of 8 keeps 16-byte alignment of the carved tensor


class Carved:
    """A tensor of `shape` inside a buffer with sentinel-filled guards."""

    def __init__(self, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        pad = (-n) % 8
        self.sentinel = 1024.0 if dtype != torch.uint8 else 0x5A
        self.buf = torch.full((n + pad + 2 * GUARD,), self.sentinel, device=DEV, dtype=dtype)
        self.t = self.buf[GUARD:GUARD + n].view(shape)
        self.n = n

    def intact(self) -> bool:
        lo, hi = self.buf[:GUARD], self.buf[GUARD + self.n:]
        return bool((lo == self.sentinel).all()) and bool((hi == self.sentinel).all())


def _p(t):
    return None if t is None else t.data_ptr()


SHAPES = [(2, 70, 72, 0), (3, 37, 20, 0), (1, 150, 64, 64), (2, 129, 192, 64), (1, 5, 8, 0)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_outputs_stay_inside_their_tensors(shape, dtype):
    from griffin_b200 import _lib
    lib = _lib.load()
    B, T, D, bw = shape
    io = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
    gen = torch.Generator(device=DEV).manual_seed(T * 31 + D)
    rnd = lambda *s: torch.randn(*s, device=DEV, generator=gen)
    x, ur, ui, br, dy = (rnd(B, T, D).to(dtype) for _ in range(5))
    lam = rnd(D) + 2.0
    h0, dh = rnd(B, D), rnd(B, D)
    w, bias = rnd(D, 4) * 0.5, rnd(D) * 0.1
    state = rnd(B, 3, D).to(dtype)
    tok = torch.zeros(B, T, device=DEV, dtype=torch.uint8)
    tok[:, 0] = 3 | 4
    tok[:, T // 2] = 3 | 4
    if T > 2:
        tok[:, T // 2 + 1] = 2
        tok[-1, T - 1] = 8
    st = torch.cuda.current_stream().cuda_stream
    nb = lib.rglru_workspace_bytes(B, T, D, io)
    guards = []

    def carve(shape_, dt=dtype):
        c = Carved(shape_, dt)
        guards.append(c)
        return c.t

    def check(rc, name):
        assert rc == 0, (name, rc)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0, name
        for i, c in enumerate(guards):
            assert c.intact(), (name, "guard", i)

    # plain scan
    y, hl, ws = carve((B, T, D)), carve((B, D), torch.float32), carve((nb,), torch.uint8)
    check(lib.rglru_fwd(_p(x), _p(ur), _p(ui), _p(lam), _p(h0), _p(tok), _p(y), _p(hl), _p(ws), nb, B, T, D, 8.0, io, st),
          "rglru_fwd")
    dx, dur, dui = carve((B, T, D)), carve((B, T, D)), carve((B, T, D))
    dlam, dh0 = carve((D,), torch.float32), carve((B, D), torch.float32)
    check(lib.rglru_bwd(_p(dy), _p(dh), _p(x), _p(ur), _p(ui), _p(lam), _p(h0), _p(tok), _p(ws), nb, _p(dx), _p(dur),
                        _p(dui), _p(dlam), _p(dh0), B, T, D, 8.0, io, st), "rglru_bwd")
    # conv folded + branch merge (covers the halo tile and the fifth tile)
    dbr = carve((B, T, D))
    check(lib.rglru_merge_fwd(_p(x), _p(w), _p(bias), _p(state), _p(ur), _p(ui), _p(br), _p(lam), _p(h0), _p(tok), _p(y),
                              _p(hl), _p(ws), nb, B, T, D, 8.0, io, st), "rglru_merge_fwd")
    check(lib.rglru_merge_bwd(_p(dy), _p(dh), _p(x), _p(w), _p(bias), _p(state), _p(ur), _p(ui), _p(br), _p(lam), _p(h0),
                              _p(tok), _p(ws), nb, _p(dx), _p(dur), _p(dui), _p(dbr), _p(dlam), _p(dh0), B, T, D, 8.0, io,
                              st), "rglru_merge_bwd")
    check(lib.rglru_conv_scan_fwd(_p(x), _p(w), _p(bias), _p(state), _p(ur), _p(ui), _p(lam), _p(h0), _p(tok), _p(y),
                                  _p(hl), _p(ws), nb, B, T, D, 8.0, io, st), "rglru_conv_scan_fwd")
    check(lib.rglru_conv_scan_bwd(_p(dy), _p(dh), _p(x), _p(w), _p(bias), _p(state), _p(ur), _p(ui), _p(lam), _p(h0),
                                  _p(tok), _p(ws), nb, _p(dx), _p(dur), _p(dui), _p(dlam), _p(dh0), B, T, D, 8.0, io, st),
          "rglru_conv_scan_bwd")
    # grouped gate layout where the shape allows it
    if bw:
        u2 = rnd(B, T, 2 * D).to(dtype)
        gbias = rnd(2 * D)
        du2 = carve((B, T, 2 * D))
        dgb = carve((2 * D,), torch.float32)
        check(lib.rglru_grouped_fwd(_p(x), _p(u2), _p(gbias), _p(br), _p(lam), _p(h0), _p(tok), _p(y), _p(hl), _p(ws), nb,
                                    B, T, D, bw, 8.0, io, st), "rglru_grouped_fwd")
        check(lib.rglru_grouped_bwd(_p(dy), _p(dh), _p(x), _p(u2), _p(gbias), _p(br), _p(lam), _p(h0), _p(tok), _p(ws), nb,
                                    _p(dx), _p(du2), _p(dbr), _p(dlam), _p(dh0), _p(dgb), B, T, D, bw, 8.0, io, st),
              "rglru_grouped_bwd")
        # the gate-bias gradient is the column sum of du (taken before rounding, rows folded in order)
        want = du2.float().sum(dim=(0, 1))
        assert float((dgb - want).norm() / want.norm().clamp_min(1e-20)) <= (1e-5 if dtype == torch.float32 else 2e-2)
    # conv alone
    xc, ns = carve((B, T, D)), carve((B, 3, D))
    check(lib.rglru_conv_fwd(_p(x), _p(w), _p(bias), _p(state), _p(tok), _p(xc), _p(ns), B, T, D, io, st), "rglru_conv_fwd")
    cb = lib.rglru_conv_bwd_workspace_bytes(B, T, D)
    cws = carve((cb,), torch.uint8)
    dw, db, dst = carve((D, 4), torch.float32), carve((D,), torch.float32), carve((B, 3, D))
    check(lib.rglru_conv_bwd(_p(dy), _p(x), _p(w), _p(state), _p(tok), _p(dx), _p(dw), _p(db), _p(dst), _p(cws), cb, B, T,
                             D, io, st), "rglru_conv_bwd")
    # raw scan (fp32 only) and decode
    if dtype == torch.float32:
        dec = torch.sigmoid(rnd(B, T, D))
        out, dd, dv = carve((B, T, D)), carve((B, T, D)), carve((B, T, D))
        check(lib.rglru_linear_scan_fwd(_p(dec), _p(x), _p(h0), _p(out), B, T, D, st), "rglru_linear_scan_fwd")
        check(lib.rglru_linear_scan_bwd(_p(dy), _p(dec), _p(h0), _p(out), _p(dd), _p(dv), _p(dh0), B, T, D, st),
              "rglru_linear_scan_bwd")
    hstate, cstate, y1 = carve((B, D), torch.float32), carve((B, 3, D)), carve((B, D))
    hstate.copy_(h0)
    cstate.copy_(state)
    x1 = x[:, 0].contiguous()
    check(lib.rglru_decode_conv(_p(x1), _p(w), _p(bias), _p(cstate), None, _p(y1), B, D, io, st), "rglru_decode_conv")
    check(lib.rglru_decode_step(_p(x1), _p(ur[:, 0].contiguous()), _p(ui[:, 0].contiguous()), _p(lam), _p(hstate), None,
                                _p(y1), B, D, 8.0, io, st), "rglru_decode_step")
    for t in (y, dx, dur, dui, dbr, xc, y1):
        assert torch.isfinite(t.float()).all()
