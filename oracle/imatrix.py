"""Importance-weighted K-quant quantization (`from_float_imatrix`) restated in scalar float32 Python - TEST INFRASTRUCTURE.

Only tests may import this file; the product's quantizer is candle_b200/csrc/host/quantize_weights.cpp.  Every operation is
one np.float32 operation in the order candle performs it:

    make_qkx3_quants   candle-core/src/quantized/utils.rs:356-466
    make_qp_quants     utils.rs:470-562
    make_qx_quants     utils.rs:62-185 (rmse_type 1, with a weight per element)
    from_float_imatrix k_quants.rs:955-1011 (Q2K), :1271-1366 (Q3K), :1602-1664 (Q4K), :1879-1957 (Q5K), :2166-2243 (Q6K)

PARITY UNPINNED: the reference holds no known-answer vector for these routines (its imatrix tests,
candle-core/tests/quantized_tests.rs:555-750, compare errors on random tensors), so this file pins nothing by itself; it is a
second, independently written statement of the same source that the compiled quantizer must agree with byte for byte.
Pure Python loops: small inputs only (a few blocks per call).
"""
from __future__ import annotations

import math
import struct

import numpy as np

F = np.float32
QK_K = 256


def _nearest_int(v) -> int:
    """`v.round() as i32`: halves away from zero, saturating, NaN -> 0."""
    v = float(v)
    if v != v:
        return 0
    r = math.floor(abs(v) + 0.5)
    r = r if v >= 0 else -r
    return max(-2 ** 31, min(2 ** 31 - 1, int(r)))


def _clamp(v: int, lo: int, hi: int) -> int:
    return lo if v < lo else hi if v > hi else v


def _f16_bits(v) -> int:
    return struct.unpack("<H", np.float16(F(v)).tobytes())[0]


def _f16_round(v):
    return F(np.float16(F(v)))


def _fsum(values):
    s = F(-0.0)
    for v in values:
        s = F(s + v)
    return s


def make_qkx3(nmax: int, x, w, rmin, rdelta, nstep: int):
    n = len(x)
    min_val, max_val = x[0], x[0]
    sum_w = w[0]
    sum_x = F(sum_w * x[0])
    for i in range(1, n):
        if x[i] < min_val:
            min_val = x[i]
        if x[i] > max_val:
            max_val = x[i]
        sum_w = F(sum_w + w[i])
        sum_x = F(sum_x + F(w[i] * x[i]))
    if min_val > 0:
        min_val = F(0.0)
    if max_val <= min_val:
        return F(0.0), F(-min_val)
    iscale = F(F(nmax) / F(max_val - min_val))
    scale = F(F(1.0) / iscale)
    best_mad = F(0.0)
    for i in range(n):
        l = _clamp(_nearest_int(F(iscale * F(x[i] - min_val))), 0, nmax)
        diff = F(F(F(scale * F(l)) + min_val) - x[i])
        best_mad = F(best_mad + F(w[i] * F(diff * diff)))
    if nstep < 1:
        return scale, F(-min_val)
    for step in range(nstep + 1):
        iscale = F(F(F(F(rmin) + F(F(rdelta) * F(step))) + F(nmax)) / F(max_val - min_val))
        sum_l = sum_l2 = sum_xl = F(0.0)
        l_aux = []
        for i in range(n):
            l = _clamp(_nearest_int(F(iscale * F(x[i] - min_val))), 0, nmax)
            l_aux.append(l)
            lf = F(l)
            sum_l = F(sum_l + F(w[i] * lf))
            sum_l2 = F(sum_l2 + F(w[i] * F(lf * lf)))
            sum_xl = F(sum_xl + F(F(w[i] * lf) * x[i]))
        d = F(F(sum_w * sum_l2) - F(sum_l * sum_l))
        if d > 0:
            this_scale = F(F(F(sum_w * sum_xl) - F(sum_x * sum_l)) / d)
            this_min = F(F(F(sum_l2 * sum_x) - F(sum_l * sum_xl)) / d)
            if this_min > 0:
                this_min = F(0.0)
                this_scale = F(sum_xl / sum_l2)
            mad = F(0.0)
            for i in range(n):
                diff = F(F(F(this_scale * F(l_aux[i])) + this_min) - x[i])
                mad = F(mad + F(w[i] * F(diff * diff)))
            if mad < best_mad:
                best_mad, scale, min_val = mad, this_scale, this_min
    return scale, F(-min_val)


def make_qp(n: int, nmax: int, x, w):
    """-> (scale, codes)."""
    mx = F(0.0)
    for v in x:
        mx = v if v > mx else mx
    if mx == 0:
        return F(0.0), [0] * n
    iscale = F(F(nmax) / mx)
    l = [_nearest_int(F(iscale * x[i])) & 0xFF for i in range(n)]
    scale = F(F(1.0) / iscale)
    best = _fsum(F(F(w[i] * F(x[i] - F(scale * F(l[i])))) * F(x[i] - F(scale * F(l[i])))) for i in range(n))
    for step in range(-4, 5):
        if step == 0:
            continue
        iscale_is = F(F(F(F(0.1) * F(step)) + F(nmax)) / mx)
        scale_is = F(F(1.0) / iscale_is)
        terms = []
        for i in range(n):
            li = min(_nearest_int(F(iscale_is * x[i])) & 0xFF, nmax)
            diff = F(x[i] - F(scale_is * F(li)))
            terms.append(F(F(w[i] * diff) * diff))
        mse = _fsum(terms)
        if mse < best:
            best, iscale = mse, iscale_is
    sumlx = suml2 = F(0.0)
    for i in range(n):
        li = min(_clamp(_nearest_int(F(iscale * x[i])), 0, 255), nmax)       # `.round() as u8` saturates
        l[i] = li
        sumlx = F(sumlx + F(F(w[i] * x[i]) * F(li)))
        suml2 = F(suml2 + F(w[i] * F(F(li) * F(li))))
    for _ in range(5):
        n_changed = 0
        for i in range(n):
            slx = F(sumlx - F(F(w[i] * x[i]) * F(l[i])))
            sl2 = F(suml2 - F(w[i] * F(F(l[i]) * F(l[i]))))
            if slx > 0 and sl2 > 0:
                new_l = min(_nearest_int(F(F(x[i] * sl2) / slx)) & 0xFF, nmax)
                if new_l != l[i]:
                    slx = F(slx + F(F(w[i] * x[i]) * F(new_l)))
                    sl2 = F(sl2 + F(w[i] * F(F(new_l) * F(new_l))))
                    if F(F(slx * slx) * suml2) > F(F(sumlx * sumlx) * sl2):
                        l[i] = new_l
                        sumlx, suml2 = slx, sl2
                        n_changed += 1
        if n_changed == 0:
            break
    return F(sumlx / suml2), l


def make_qx(n: int, nmax: int, x, qw):
    """-> (scale, codes + nmax)."""
    mx, amax = F(0.0), F(0.0)
    for v in x:
        if abs(v) > amax:
            amax, mx = F(abs(v)), v
    if amax == 0:
        return F(0.0), [0] * n
    iscale = F(F(-nmax) / mx)
    ls = [0] * n
    sumlx = suml2 = F(0.0)
    for i in range(n):
        l = _clamp(_nearest_int(F(iscale * x[i])), -nmax, nmax - 1)
        ls[i] = l + nmax
        sumlx = F(sumlx + F(F(qw[i] * x[i]) * F(l)))
        suml2 = F(suml2 + F(F(qw[i] * F(l)) * F(l)))
    scale = F(sumlx / suml2)
    best = F(scale * sumlx)
    for _ in range(3):
        isc = F(F(1.0) / scale)
        slx = sl2 = F(0.0)
        changed = False
        for i in range(n):
            l = _clamp(_nearest_int(F(isc * x[i])), -nmax, nmax - 1)
            if l + nmax != ls[i]:
                changed = True
            slx = F(slx + F(F(qw[i] * x[i]) * F(l)))
            sl2 = F(sl2 + F(F(qw[i] * F(l)) * F(l)))
        if not changed or sl2 == 0 or F(slx * slx) <= F(best * sl2):
            break
        for i in range(n):
            ls[i] = nmax + _clamp(_nearest_int(F(isc * x[i])), -nmax, nmax - 1)
        sumlx, suml2 = slx, sl2
        scale = F(sumlx / suml2)
        best = F(scale * sumlx)
    for _ in range(5):
        n_changed = 0
        for i in range(n):
            l = ls[i] - nmax
            slx = F(sumlx - F(F(qw[i] * x[i]) * F(l)))
            if slx > 0:
                sl2 = F(suml2 - F(F(qw[i] * F(l)) * F(l)))
                new_l = _clamp(_nearest_int(F(F(x[i] * sl2) / slx)), -nmax, nmax - 1)
                if new_l != l:
                    slx = F(slx + F(F(qw[i] * x[i]) * F(new_l)))
                    sl2 = F(sl2 + F(F(qw[i] * F(new_l)) * F(new_l)))
                    if sl2 > 0 and F(F(slx * slx) * suml2) > F(F(sumlx * sumlx) * sl2):
                        ls[i] = nmax + new_l
                        sumlx, suml2 = slx, sl2
                        scale = F(sumlx / suml2)
                        best = F(scale * sumlx)
                        n_changed += 1
        if n_changed == 0:
            break
    return scale, ls


def _weights(xs, imp, sigma2):
    w = [F(imp[i] * np.sqrt(F(sigma2 + F(xs[i] * xs[i])))) for i in range(len(xs))]
    return w, _fsum(w)


def _scale_min_k4(j, q):
    if j < 4:
        return q[j] & 63, q[j + 4] & 63
    return (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4), (q[j + 4] >> 4) | ((q[j] >> 6) << 4)


def _pack_k4(ls, lm):
    sc = [0] * 12
    for j in range(8):
        a, c = min(ls[j], 63), min(lm[j], 63)
        if j < 4:
            sc[j], sc[j + 4] = a, c
        else:
            sc[j + 4] = (a & 0xF) | ((c & 0xF) << 4)
            sc[j - 4] |= (a >> 4) << 6
            sc[j] |= (c >> 4) << 6
    return sc


def _block_q45k(x, imp, bits):
    levels = (1 << bits) - 1
    sigma2 = F(F(F(2.0) * _fsum(F(v * v) for v in x)) / F(QK_K))
    scales, mins, sw = [], [], []
    for j in range(8):
        xs = x[32 * j:32 * j + 32]
        w, s = _weights(xs, imp[32 * j:32 * j + 32], sigma2)
        sw.append(s)
        sc, mn = make_qkx3(levels, xs, w, -0.9, 0.05, 36)
        scales.append(sc), mins.append(mn)
    d_block, ls = make_qp(8, 63, scales, sw)
    m_block, lm = make_qp(8, 63, mins, sw)
    sc12 = _pack_k4(ls, lm)
    d16, m16 = _f16_bits(d_block), _f16_bits(m_block)
    dq, mq = _f16_round(d_block), _f16_round(m_block)
    l = [0] * QK_K
    for j in range(8):
        sc, m = _scale_min_k4(j, sc12)
        d = F(dq * F(sc))
        if d != 0:
            dm = F(mq * F(m))
            for ii in range(32):
                l[32 * j + ii] = _clamp(_nearest_int(F(F(x[32 * j + ii] + dm) / d)), 0, levels)
    qh, qs = [0] * 32, [0] * 128
    for g in range(4):
        for j in range(32):
            l1, l2 = l[64 * g + j], l[64 * g + j + 32]
            if l1 > 15:
                l1 -= 16
                qh[j] |= 1 << (2 * g)
            if l2 > 15:
                l2 -= 16
                qh[j] |= 2 << (2 * g)
            qs[32 * g + j] = l1 | (l2 << 4)
    head = struct.pack("<HH", d16, m16) + bytes(sc12)
    return head + (bytes(qh) if bits == 5 else b"") + bytes(qs)


def _block_q2k(x, imp):
    sigma2 = F(_fsum(F(v * v) for v in x) / F(QK_K))
    scales, mins, sw = [], [], []
    for j in range(16):
        xs = x[16 * j:16 * j + 16]
        w, s = _weights(xs, imp[16 * j:16 * j + 16], sigma2)
        sw.append(s)
        sc, mn = make_qkx3(3, xs, w, -0.9, 0.05, 36)
        scales.append(sc), mins.append(mn)
    d_block, ls = make_qp(16, 15, scales, sw)
    m_block, lm = make_qp(16, 15, mins, sw)
    dq, mq = _f16_round(d_block), _f16_round(m_block)
    sc = [(ls[j] | (lm[j] << 4)) & 0xFF for j in range(16)]
    big = [0] * QK_K
    for j in range(16):
        d = F(dq * F(sc[j] & 0xF))
        if d == 0:
            continue
        dm = F(mq * F(sc[j] >> 4))
        for ii in range(16):
            big[16 * j + ii] = _clamp(_nearest_int(F(F(x[16 * j + ii] + dm) / d)), 0, 3)
    qs = [0] * 64
    for j in range(0, QK_K, 128):
        for t in range(32):
            qs[j // 4 + t] = big[j + t] | (big[j + t + 32] << 2) | (big[j + t + 64] << 4) | (big[j + t + 96] << 6)
    return bytes(sc) + bytes(qs) + struct.pack("<HH", _f16_bits(d_block), _f16_bits(m_block))


def _block_q3k(x, imp):
    sigma2 = F(F(F(2.0) * _fsum(F(v * v) for v in x)) / F(QK_K))
    scales, sw, l = [], [], [0] * QK_K
    for j in range(16):
        xs = x[16 * j:16 * j + 16]
        w, s = _weights(xs, imp[16 * j:16 * j + 16], sigma2)
        sw.append(s)
        sc, codes = make_qx(16, 4, xs, w)
        scales.append(sc)
        l[16 * j:16 * j + 16] = codes
    d_block, ls = make_qx(16, 32, scales, sw)
    dq = _f16_round(d_block)
    sc12 = [0] * 12
    for j in range(16):
        lv = ls[j]
        if j < 8:
            sc12[j] = lv & 0xF
        else:
            sc12[j - 8] |= (lv & 0xF) << 4
        sc12[j % 4 + 8] |= ((lv >> 4) << (2 * (j // 4))) & 0xFF
    for j in range(16):
        lo = (sc12[j] & 0xF) if j < 8 else (sc12[j - 8] >> 4)
        sc = (lo | (((sc12[8 + j % 4] >> (2 * (j // 4))) & 3) << 4)) - 32
        d = F(dq * F(sc))
        if d != 0:
            for ii in range(16):
                l[16 * j + ii] = _clamp(_nearest_int(F(x[16 * j + ii] / d)), -4, 3) + 4
    hmask = [0] * 32
    m, hm = 0, 1
    for e in range(QK_K):
        if l[e] > 3:
            hmask[m] |= hm
            l[e] -= 4
        m += 1
        if m == QK_K // 8:
            m, hm = 0, hm << 1
    qs = [0] * 64
    for j in range(0, QK_K, 128):
        for t in range(32):
            qs[j // 4 + t] = l[j + t] | (l[j + t + 32] << 2) | (l[j + t + 64] << 4) | (l[j + t + 96] << 6)
    return bytes(hmask) + bytes(qs) + bytes(sc12) + struct.pack("<H", _f16_bits(d_block))


def _block_q6k(x, imp, carry):
    """`carry`: the 256 codes left by the previous block (the reference reuses one array across blocks)."""
    l = carry
    scales = []
    max_scale = max_abs = F(0.0)
    for j in range(16):
        s, codes = make_qx(16, 32, x[16 * j:16 * j + 16], imp[16 * j:16 * j + 16])
        l[16 * j:16 * j + 16] = codes
        scales.append(s)
        if abs(s) > max_abs:
            max_abs, max_scale = F(abs(s)), s
    with np.errstate(divide="ignore", invalid="ignore"):
        iscale = F(F(-128.0) / max_scale)
        d_val = F(F(1.0) / iscale)
        dq = _f16_round(d_val)
        sc = []
        for s in scales:
            v = min(_nearest_int(F(iscale * s)), 127) & 0xFF
            sc.append(v - 256 if v > 127 else v)
    for j in range(16):
        d = F(dq * F(sc[j]))
        if d == 0:
            continue
        for ii in range(16):
            l[16 * j + ii] = _clamp(_nearest_int(F(x[16 * j + ii] / d)), -32, 31) + 32
    ql, qh = [0] * 128, [0] * 64
    for j in range(0, QK_K, 128):
        for t in range(32):
            a0, a1, a2, a3 = l[j + t], l[j + t + 32], l[j + t + 64], l[j + t + 96]
            ql[j // 2 + t] = (a0 & 0xF) | ((a2 & 0xF) << 4)
            ql[j // 2 + t + 32] = (a1 & 0xF) | ((a3 & 0xF) << 4)
            qh[j // 4 + t] = (a0 >> 4) | ((a1 >> 4) << 2) | ((a2 >> 4) << 4) | ((a3 >> 4) << 6)
    return bytes(ql) + bytes(qh) + bytes(v & 0xFF for v in sc) + struct.pack("<H", _f16_bits(d_val))


def quantize_imatrix(name: str, x, imatrix) -> bytes:
    """`x`: f32 values, flattened rows of `len(imatrix)` elements; `name`: Q2K, Q3K, Q4K, Q5K or Q6K."""
    x = [F(v) for v in np.asarray(x, dtype=np.float32).reshape(-1)]
    imatrix = [F(v) for v in np.asarray(imatrix, dtype=np.float32).reshape(-1)]
    per_row = len(imatrix) // QK_K
    out = b""
    carry = [0] * QK_K
    with np.errstate(all="ignore"):        # a sub-block whose weighted codes are all zero gives 0 / 0, as in the reference
        return _quantize_blocks(name, x, imatrix, per_row, out, carry)


def _quantize_blocks(name, x, imatrix, per_row, out, carry) -> bytes:
    for ib in range(len(x) // QK_K):
        xb = x[ib * QK_K:(ib + 1) * QK_K]
        imp = imatrix[(ib % per_row) * QK_K:(ib % per_row + 1) * QK_K]
        if name == "Q4K":
            out += _block_q45k(xb, imp, 4)
        elif name == "Q5K":
            out += _block_q45k(xb, imp, 5)
        elif name == "Q2K":
            out += _block_q2k(xb, imp)
        elif name == "Q3K":
            out += _block_q3k(xb, imp)
        elif name == "Q6K":
            out += _block_q6k(xb, imp, carry)
        else:
            raise ValueError(f"`from_float_imatrix` is unimplemented for {name}")
    return out
