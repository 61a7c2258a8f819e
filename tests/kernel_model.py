"""Lane-level numpy model of the GEMV kernel's data path (test infrastructure).

It reads a packed blob exactly the way the CUDA kernel does -- the same work split between
CTAs, phases, warps and lanes, the same fragment addresses, the same activation-fragment
permutation, the same partial-slot and part-count arithmetic -- and accumulates in fp64.  It
needs no GPU, so the packer, the layout header and the scheduling arithmetic are checked on
CPU against the oracle before the kernel ever runs.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle as O

PMAX = 8
PHASE_UNITS = 16
HEADER = 256


def _hdr(blob: np.ndarray):
    fmt = int(blob[8:12].view(np.uint32)[0])
    N, K, n_panels, units = (int(v) for v in blob[16:48].view(np.int64))
    unit_bytes = int(blob[48:52].view(np.uint32)[0])
    ts = float(blob[56:60].view(np.float32)[0])
    aux_bytes = int(blob[64:72].view(np.uint64)[0])
    return fmt, N, K, n_panels, units, unit_bytes, ts, aux_bytes


def items_of_cta(cta: int, grid: int, total: int, units: int, n_panels: int):
    pos = (cta * total) // grid
    end = ((cta + 1) * total) // grid
    out = []
    while pos < end:
        vp, u0 = divmod(pos, units)
        left = end - pos
        if u0 != 0 or left < units:
            u1 = min(units, u0 + left)
            out.append(dict(vp=vp, np=1, u0=u0, u1=u1, partial=1, start=pos))
            pos += u1 - u0
        else:
            npan = min(left // units, n_panels - (vp % n_panels), PMAX)
            out.append(dict(vp=vp, np=npan, u0=0, u1=units, partial=0, start=pos))
            pos += npan * units
    return out


def cta_of(idx: int, total: int, grid: int) -> int:
    return ((idx + 1) * grid - 1) // total


def part_slot(c: int, vp: int, units: int, total: int, grid: int) -> int:
    a = (c * total) // grid
    ov = max(a, vp * units)
    return 2 * c + (0 if ov == a else 1)


def _a_fragment(unit: np.ndarray, fmt: int, lane: int):
    """The four tiles' A registers of one lane as values: a[T][jb][h] (already scaled for NVFP4)."""
    g = lane >> 2
    a = np.zeros((4, 4, 2), dtype=np.float64)
    if fmt == 1:
        words = unit[lane * 16: lane * 16 + 16].reshape(4, 4)  # [T][byte]
        sc = O.np_e4m3_decode(unit[512 + g * 8: 512 + g * 8 + 8]).astype(np.float64)  # row g blk0..3, row g+8 blk0..3
        for T in range(4):
            pr = T >> 1
            for jb in range(4):
                byte = int(words[T, jb])
                rowhi = jb & 1
                for h in range(2):
                    code = (byte >> 4) if h else (byte & 15)
                    a[T, jb, h] = float(O.E2M1_VALUES[code]) * sc[rowhi * 4 + 2 * pr + h]
    else:
        for T in range(4):
            base = (T >> 1) * 512 + lane * 16 + (T & 1) * 8
            for jb in range(4):
                for h in range(2):
                    a[T, jb, h] = float(O.np_e4m3_decode(unit[base + 2 * jb + h: base + 2 * jb + h + 1])[0])
    return a


def model_gemv(blob: np.ndarray, x_bf16: np.ndarray, grid: int, chan_scale=None):
    """Returns y f64 [B][N] computed the way the kernel walks the blob, plus bookkeeping."""
    fmt, N, K, n_panels, units, unit_bytes, ts, aux_bytes = _hdr(blob)
    payload = blob[HEADER + aux_bytes:]
    chan = blob[HEADER:HEADER + aux_bytes].view(np.float32) if fmt == 2 else None
    B = x_bf16.shape[0]
    x = O.bf16_decode(x_bf16).astype(np.float64)
    total = n_panels * units
    grid = min(grid, total)
    y = np.full((B, N), np.nan)
    ws = {}
    counters = {}
    covered = np.zeros(total, dtype=np.int32)
    max_parts = 0
    for cta in range(grid):
        for it in items_of_cta(cta, grid, total, units, n_panels):
            c = np.zeros((it["np"], 8, 32, 4))  # [panel][warp][lane][reg]
            f0, f1 = it["u0"] // PHASE_UNITS, (it["u1"] - 1) // PHASE_UNITS
            for f in range(f0, f1 + 1):
                ua, ub = max(it["u0"], f * PHASE_UNITS), min(it["u1"], (f + 1) * PHASE_UNITS)
                # converter: fragment buffer of the phase, f16x2 words as (lo, hi) value pairs
                xbuf = np.zeros((PHASE_UNITS, 2, 32, 4, 2))
                for b in range(B):
                    for i in range(128):
                        q, pp, t = i >> 3, (i >> 2) & 1, i & 3
                        u = f * PHASE_UNITS + q
                        if not (ua <= u < ub):
                            continue
                        k = u * 64 + pp * 32 + 4 * t
                        va = x[b, k:k + 4] if k < K else np.zeros(4)
                        vb = x[b, k + 16:k + 20] if k + 16 < K else np.zeros(4)
                        for wd in range(4):
                            xbuf[q, pp, 4 * b + t, wd, 0] = va[wd] if wd < len(va) else 0.0
                            xbuf[q, pp, 4 * b + t, wd, 1] = vb[wd] if wd < len(vb) else 0.0
                for pl in range(it["np"]):
                    vp = it["vp"] + pl
                    panel = vp % n_panels
                    covered[vp * units + ua: vp * units + ub] += 1
                    off = (panel * units + ua) * unit_bytes
                    stage = payload[off: off + (ub - ua) * unit_bytes]
                    for w in range(8):
                        for qq in (2 * w, 2 * w + 1):
                            u = f * PHASE_UNITS + qq
                            if not (ua <= u < ub):
                                continue
                            unit = stage[(u - ua) * unit_bytes:(u - ua + 1) * unit_bytes]
                            # whole-tile form
                            A = np.zeros((4, 16, 16))
                            Bm = np.zeros((4, 16, 8))
                            for lane in range(32):
                                a = _a_fragment(unit, fmt, lane)
                                g, t = lane >> 2, lane & 3
                                for T in range(4):
                                    for jb in range(4):
                                        row = g + 8 * (jb & 1)
                                        r = jb >> 1
                                        for h in range(2):
                                            A[T, row, 2 * t + 8 * r + h] = a[T, jb, h]
                                    pr, sub = T >> 1, T & 1
                                    for r in range(2):
                                        for h in range(2):
                                            Bm[T, 2 * t + 8 * r + h, g] = xbuf[qq, pr, lane, 2 * sub + r, h]
                            Ct = np.einsum("tij,tjk->ik", A, Bm)
                            for lane in range(32):
                                g, t = lane >> 2, lane & 3
                                c[pl, w, lane] += [Ct[g, 2 * t], Ct[g, 2 * t + 1], Ct[g + 8, 2 * t], Ct[g + 8, 2 * t + 1]]
            # flush
            for pl in range(it["np"]):
                v = c[pl].sum(axis=0) * ts  # [lane][4]
                vp = it["vp"] + pl
                panel = vp % n_panels
                if not it["partial"]:
                    _store(y, v, panel, N, B, chan)
                else:
                    c_lo = cta_of(vp * units, total, grid)
                    c_hi = cta_of((vp + 1) * units - 1, total, grid)
                    nparts = c_hi - c_lo + 1
                    max_parts = max(max_parts, nparts)
                    slot = part_slot(cta, vp, units, total, grid)
                    assert slot not in ws, "workspace slot reused within a launch"
                    ws[slot] = v
                    counters[vp] = counters.get(vp, 0) + 1
                    if counters[vp] == nparts:
                        acc = None
                        for cc in range(c_lo, c_hi + 1):
                            part = ws[part_slot(cc, vp, units, total, grid)]
                            acc = part.copy() if acc is None else acc + part
                        _store(y, acc, panel, N, B, chan)
                        counters[vp] = 0
    assert (covered == 1).all(), "every (panel, unit) block must be consumed exactly once"
    assert all(v == 0 for v in counters.values()), "a split panel never got all its parts"
    return y, dict(max_parts=max_parts, slots=len(ws))


def _store(y, v, panel, N, B, chan):
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for i in range(4):
            col = 2 * t + (i & 1)
            n = panel * 16 + g + (8 if i & 2 else 0)
            if col < B and n < N:
                y[col, n] = v[lane, i] * (float(chan[n]) if chan is not None else 1.0)
