"""Seeded synthetic GGUF tensors (stand-ins for real model files, none of which is needed).

Two generators, both producing raw GGUF block bytes uint8 [n_out, (K/256) * bytes_per_256]:

* random_blocks — the reference's own test method: every bit pattern of the quantised fields is
  legal, only the fp16 d / dmin fields are forced to small finite values
  (gguf-plugin/gluon/kq_ref.py:94-112, gguf-plugin/test_gluon_wide_gpu.py:47-57).  Runs on any torch
  device, so a 10 GB layer stack is generated on the GPU in seconds.
* encode — straightforward round-to-nearest encoders written from each format's decode equations
  (per-group affine or symmetric fit; nearest codebook entry for IQ4; nearest grid point by brute
  force for IQ3_S), applied to seeded N(0, sigma) weights so field statistics resemble a real tensor.
  They are NOT ggml's search-based quantizers; parity is defined on the produced bytes.
"""
from __future__ import annotations

import numpy as np
import torch

from . import formats as F

# byte offsets of the fp16 d (and dmin) fields inside one GGML block
_D_OFF = {F.Q4_0: (0,), F.Q5_0: (0,), F.Q8_0: (0,), F.IQ4_NL: (0,), F.Q2_K: (80, 82), F.Q3_K: (108,),
          F.Q4_K: (0, 2), F.Q5_K: (0, 2), F.Q6_K: (208,), F.IQ3_S: (0,), F.IQ4_XS: (0,),
          F.IQ3_XXS: (0,), F.IQ2_XXS: (0,), F.IQ2_XS: (0,), F.IQ2_S: (0,), F.IQ1_M: ()}


def random_blocks(n_out: int, k: int, wtype: int, seed: int, device="cpu", d_exp: int = -6) -> torch.Tensor:
    """Random valid rows of the type: uniform random bytes, d = U(0.25, 1) * 2^d_exp, dmin = U(0.25, 1) * 2^(d_exp - 2)."""
    wpb, bpb = F.GGML_BLOCK[wtype]
    if k % F.QK:
        raise ValueError(f"K={k} is not a multiple of {F.QK}")
    nblk = k // wpb
    g = torch.Generator(device=device).manual_seed(int(seed))
    raw = torch.randint(0, 256, (n_out, nblk, bpb), dtype=torch.uint8, device=device, generator=g)
    for i, off in enumerate(_D_OFF[wtype]):
        u = torch.rand((n_out, nblk), device=device, generator=g) * 0.75 + 0.25
        val = (u * (2.0 ** d_exp if i == 0 else 2.0 ** (d_exp - 2))).to(torch.float16)
        raw[:, :, off:off + 2] = val.view(torch.uint8).reshape(n_out, nblk, 2)
    if wtype == F.IQ1_M:
        # the fp16 d of IQ1_M lives in the top nibbles of the four scale halfwords (bytes 49, 51, 53, 55)
        u = torch.rand((n_out, nblk), device=device, generator=g) * 0.75 + 0.25
        bits = (u * 2.0 ** d_exp).to(torch.float16).view(torch.int16).to(torch.int32) & 0xFFFF
        for i in range(4):
            hi = raw[:, :, 49 + 2 * i].to(torch.int32)
            raw[:, :, 49 + 2 * i] = ((hi & 0x0F) | (((bits >> (4 * i)) & 0xF) << 4)).to(torch.uint8)
    return raw.reshape(n_out, nblk * bpb)


def gaussian_weights(n_out: int, k: int, seed: int, sigma: float = 0.02) -> np.ndarray:
    g = torch.Generator().manual_seed(int(seed))
    return (torch.randn((n_out, k), generator=g, dtype=torch.float32) * sigma).numpy()


def activations(m: int, k: int, seed: int | None = None, device="cpu", sigma: float = 1.0) -> torch.Tensor:
    """bf16 N(0, sigma) activations [m, k], seed 100 + m unless given (the reference's pattern,
    gguf-plugin/test_gluon_kq_gpu.py:131)."""
    g = torch.Generator().manual_seed(100 + m if seed is None else int(seed))
    return (torch.randn((m, k), generator=g, dtype=torch.float32) * sigma).to(torch.bfloat16).to(device)


# ---- encoders -----------------------------------------------------------------------------------

def _f16(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    h = x.astype(np.float16)
    return h.astype(np.float32), h.view(np.uint8).reshape(*x.shape, 2)


def _safe_div(a, b):
    return np.divide(a, b, out=np.zeros_like(a, dtype=np.float32), where=b != 0)


def _pack_scale_min_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """sc, mn uint8 [n, 8] (6-bit) -> the 12 packed bytes of Q4_K / Q5_K."""
    s = np.zeros(sc.shape[:-1] + (12,), np.uint8)
    for j in range(4):
        s[..., j] = (sc[..., j] & 63) | ((sc[..., j + 4] >> 4) << 6)
        s[..., j + 4] = (mn[..., j] & 63) | ((mn[..., j + 4] >> 4) << 6)
        s[..., j + 8] = (sc[..., j + 4] & 0xF) | ((mn[..., j + 4] & 0xF) << 4)
    return s


def _affine_groups(w: np.ndarray, group: int, qmax: int, smax: int):
    """w [n, 256] -> (d, dmin fp32 [n,1] (fp16-rounded), their bytes, sc, mn uint8 [n, G], q uint8 [n, 256])
    for w ~ d*sc*q - dmin*mn with mn >= 0."""
    n = w.shape[0]
    G = F.QK // group
    wg = w.reshape(n, G, group)
    lo = np.minimum(wg.min(-1), 0.0)
    hi = np.maximum(wg.max(-1), 0.0)
    scale = (hi - lo) / qmax
    d, db = _f16(scale.max(-1, keepdims=True) / smax)
    dm, dmb = _f16((-lo).max(-1, keepdims=True) / smax)
    sc = np.clip(np.rint(_safe_div(scale, d)), 0, smax).astype(np.uint8)
    mn = np.clip(np.rint(_safe_div(-lo, dm)), 0, smax).astype(np.uint8)
    step = (d * sc)[..., None]
    q = np.clip(np.rint(_safe_div(wg + (dm * mn)[..., None], np.broadcast_to(step, wg.shape).copy())), 0, qmax)
    return d, db, dm, dmb, sc, mn, q.astype(np.uint8).reshape(n, F.QK)


def _enc_q4_k(w):
    n = w.shape[0]
    _, db, _, dmb, sc, mn, q = _affine_groups(w, 32, 15, 63)
    q = q.reshape(n, 4, 2, 32)
    qs = (q[:, :, 0] | (q[:, :, 1] << 4)).reshape(n, 128)
    return np.concatenate([db.reshape(n, 2), dmb.reshape(n, 2), _pack_scale_min_k4(sc, mn), qs], axis=1)


def _enc_q5_k(w):
    n = w.shape[0]
    _, db, _, dmb, sc, mn, q = _affine_groups(w, 32, 31, 63)
    q8 = q.reshape(n, 8, 32)
    qh = np.zeros((n, 32), np.uint8)
    for ib in range(8):
        qh |= ((q8[:, ib] >> 4) & 1) << ib
    ql = (q8 & 0xF).reshape(n, 4, 2, 32)
    qs = (ql[:, :, 0] | (ql[:, :, 1] << 4)).reshape(n, 128)
    return np.concatenate([db.reshape(n, 2), dmb.reshape(n, 2), _pack_scale_min_k4(sc, mn), qh, qs], axis=1)


def _enc_q2_k(w):
    n = w.shape[0]
    _, db, _, dmb, sc, mn, q = _affine_groups(w, 16, 3, 15)
    scales = (sc | (mn << 4)).astype(np.uint8)
    q = q.reshape(n, 2, 4, 32)
    qs = np.zeros((n, 2, 32), np.uint8)
    for t in range(4):
        qs |= q[:, :, t] << (2 * t)
    return np.concatenate([scales, qs.reshape(n, 64), db.reshape(n, 2), dmb.reshape(n, 2)], axis=1)


def _sym_groups(w, group, qlo, qhi, smax):
    """w ~ d * sc * q, sc in [0, smax], q in [qlo, qhi]."""
    n = w.shape[0]
    G = F.QK // group
    wg = w.reshape(n, G, group)
    scale = np.abs(wg).max(-1) / max(abs(qlo), abs(qhi))
    d, db = _f16(scale.max(-1, keepdims=True) / smax)
    sc = np.clip(np.rint(_safe_div(scale, d)), 0, smax).astype(np.int32)
    step = np.broadcast_to((d * sc)[..., None], wg.shape).copy()
    q = np.clip(np.rint(_safe_div(wg, step)), qlo, qhi).astype(np.int32)
    return db, sc, q.reshape(n, F.QK)


def _enc_q3_k(w):
    n = w.shape[0]
    db, sc, q = _sym_groups(w, 16, -4, 3, 31)
    s6 = (sc + 32).astype(np.uint8)                       # stored 6-bit, value - 32
    scales = np.zeros((n, 12), np.uint8)
    for i in range(16):
        scales[:, i % 8] |= (s6[:, i] & 0xF) << (4 * (i // 8))
        scales[:, 8 + i % 4] |= ((s6[:, i] >> 4) & 3) << (2 * (i // 4))
    u = (q + 4).astype(np.uint8)                          # 0..7: low 2 bits in qs, bit 2 in hmask
    u = u.reshape(n, 2, 4, 32)
    qs = np.zeros((n, 2, 32), np.uint8)
    hmask = np.zeros((n, 32), np.uint8)
    for nn in range(2):
        for j in range(4):
            qs[:, nn] |= (u[:, nn, j] & 3) << (2 * j)
            hmask |= ((u[:, nn, j] >> 2) & 1) << (4 * nn + j)
    return np.concatenate([hmask, qs.reshape(n, 64), scales, db.reshape(n, 2)], axis=1)


def _enc_q6_k(w):
    n = w.shape[0]
    db, sc, q = _sym_groups(w, 16, -32, 31, 127)
    u = (q + 32).astype(np.uint8).reshape(n, 2, 4, 32)    # [half, t, p]
    ql = np.zeros((n, 2, 64), np.uint8)
    qh = np.zeros((n, 2, 32), np.uint8)
    for t in range(4):
        ql[:, :, 32 * (t & 1):32 * (t & 1) + 32] |= (u[:, :, t] & 0xF) << (4 * (t >> 1))
        qh |= ((u[:, :, t] >> 4) & 3) << (2 * t)
    return np.concatenate([ql.reshape(n, 128), qh.reshape(n, 64), sc.astype(np.int8).view(np.uint8), db.reshape(n, 2)], axis=1)


def _kvalues() -> np.ndarray:
    from gguf.quants import IQ4_NL

    return np.array(IQ4_NL.kvalues, dtype=np.float32)


def _nearest_kv(x: np.ndarray) -> np.ndarray:
    kv = _kvalues()
    return np.abs(x[..., None] - kv).argmin(-1).astype(np.uint8)


def _enc_iq4_nl(w):
    n = w.shape[0]
    wb = w.reshape(n, 8, 32)
    d, db = _f16(np.abs(wb).max(-1, keepdims=True) / 127.0)
    idx = _nearest_kv(_safe_div(wb, np.broadcast_to(d, wb.shape).copy()))
    qs = idx[..., :16] | (idx[..., 16:] << 4)
    return np.concatenate([db.reshape(n, 8, 2), qs], axis=-1).reshape(n, 8 * 18)


def _enc_iq4_xs(w):
    n = w.shape[0]
    wb = w.reshape(n, 8, 32)
    scale = np.abs(wb).max(-1) / 127.0
    d, db = _f16(scale.max(-1, keepdims=True) / 31.0)
    ls = np.clip(np.rint(_safe_div(scale, d)), 0, 31).astype(np.int32)
    step = np.broadcast_to((d * ls)[..., None], wb.shape).copy()
    idx = _nearest_kv(_safe_div(wb, step))
    l6 = (ls + 32).astype(np.uint16)
    sh = np.zeros((n,), np.uint16)
    sl = np.zeros((n, 4), np.uint8)
    for ib in range(8):
        sh |= ((l6[:, ib] >> 4) & 3) << (2 * ib)
        sl[:, ib >> 1] |= (l6[:, ib] & 0xF).astype(np.uint8) << (4 * (ib & 1))
    qs = (idx[..., :16] | (idx[..., 16:] << 4)).reshape(n, 128)
    return np.concatenate([db.reshape(n, 2), sh.view(np.uint8).reshape(n, 2), sl, qs], axis=1)


def _enc_iq3_s(w):
    from gguf.quants import IQ3_S

    IQ3_S.init_grid()
    grid = IQ3_S.grid.reshape(512, 4).astype(np.float32)
    n = w.shape[0]
    wb = w.reshape(n, 8, 32)
    db_t = np.abs(wb).max(-1) / 15.0
    d, dbytes = _f16(db_t.max(-1, keepdims=True) / 31.0)
    s = np.clip(np.rint((_safe_div(db_t, d) - 1.0) / 2.0), 0, 15).astype(np.uint8)
    step = np.broadcast_to((d * (1 + 2 * s.astype(np.float32)))[..., None], wb.shape).copy()
    mag = _safe_div(np.abs(wb), step).reshape(n * 64, 4)
    idx = np.empty(n * 64, np.int32)
    for i in range(0, n * 64, 4096):
        c = mag[i:i + 4096]
        idx[i:i + 4096] = ((c[:, None, :] - grid[None]) ** 2).sum(-1).argmin(-1)
    idx = idx.reshape(n, 8, 8)
    qs = (idx & 0xFF).astype(np.uint8).reshape(n, 64)
    qh = np.zeros((n, 8), np.uint8)
    for k in range(8):
        qh |= ((idx[:, :, k] >> 8) & 1).astype(np.uint8) << k
    neg = (wb < 0).reshape(n, 8, 4, 8).astype(np.uint8)
    signs = np.zeros((n, 8, 4), np.uint8)
    for b in range(8):
        signs |= neg[..., b] << b
    scales = (s[:, 0::2] | (s[:, 1::2] << 4)).astype(np.uint8)
    return np.concatenate([dbytes.reshape(n, 2), qs, qh, signs.reshape(n, 32), scales], axis=1)


def _nearest_grid(mag: np.ndarray, grid: np.ndarray) -> np.ndarray:
    """Index of the nearest grid row for every row of mag [n, e]."""
    idx = np.empty(mag.shape[0], np.int32)
    g2 = (grid ** 2).sum(-1)
    for i in range(0, mag.shape[0], 8192):
        c = mag[i:i + 8192]
        idx[i:i + 8192] = (g2[None] - 2.0 * c @ grid.T).argmin(-1)
    return idx


def _even_signs(wg: np.ndarray) -> np.ndarray:
    """Sign masks (bit j set: weight j negative) of groups of eight with an even number of set bits, as the 7-bit sign index
    plus parity can express: a group with an odd number of negatives has its smallest magnitude's sign flipped."""
    neg = wg < 0
    odd = neg.sum(-1) % 2 == 1
    flip = np.abs(wg).argmin(-1)
    rows = np.nonzero(odd)[0]
    neg[rows, flip[rows]] ^= True
    mask = np.zeros(wg.shape[0], np.uint8)
    for j in range(8):
        mask |= neg[:, j].astype(np.uint8) << j
    return mask


def _enc_iq3_xxs(w):
    """d | qs[64] | u32[8]: weight = d (2 s + 1) / 4 x magnitude x sign, four magnitudes per grid index, the sign mask of a
    group of eight stored as its low seven bits (gguf-plugin/gluon/iq3xxs.py:5-12)."""
    from gguf.quants import IQ3_XXS

    IQ3_XXS.init_grid()
    grid = IQ3_XXS.grid.reshape(256, 4).astype(np.float32)
    n = w.shape[0]
    wb = w.reshape(n, 8, 32)
    step_t = np.abs(wb).max(-1) / 48.0
    d, dbytes = _f16(step_t.max(-1, keepdims=True) * 4.0 / 31.0)
    s = np.clip(np.rint((_safe_div(step_t * 4.0, d) - 1.0) / 2.0), 0, 15).astype(np.uint32)
    step = np.broadcast_to((d * (2 * s.astype(np.float32) + 1) / 4.0)[..., None], wb.shape)
    idx = _nearest_grid(_safe_div(np.abs(wb), step).reshape(n * 64, 4), grid).reshape(n, 64)
    signs = (_even_signs(wb.reshape(n * 32, 8)) & 0x7F).astype(np.uint32).reshape(n, 8, 4)
    word = signs[..., 0] | (signs[..., 1] << 7) | (signs[..., 2] << 14) | (signs[..., 3] << 21) | (s << 28)
    return np.concatenate([dbytes.reshape(n, 2), idx.astype(np.uint8), word.astype("<u4").view(np.uint8).reshape(n, 32)], axis=1)


def _enc_iq2(w, wtype):
    """IQ2_XXS / IQ2_XS / IQ2_S: weight = d (2 s + 1) / 8 x magnitude x sign, eight magnitudes per grid index; the scale
    is per 32 weights (IQ2_XXS) or per 16; IQ2_XXS and IQ2_XS store seven sign bits per group of eight
    (gguf-plugin/gluon/iq2.py:6-23)."""
    import gguf.quants as gq

    cls = {F.IQ2_XXS: gq.IQ2_XXS, F.IQ2_XS: gq.IQ2_XS, F.IQ2_S: gq.IQ2_S}[wtype]
    cls.init_grid()
    grid = cls.grid.reshape(-1, 8).astype(np.float32)
    n = w.shape[0]
    grp = 32 if wtype == F.IQ2_XXS else 16
    wb = w.reshape(n, 256 // grp, grp)
    step_t = np.abs(wb).max(-1) / 36.0
    d, dbytes = _f16(step_t.max(-1, keepdims=True) * 8.0 / 31.0)
    s = np.clip(np.rint((_safe_div(step_t * 8.0, d) - 1.0) / 2.0), 0, 15).astype(np.uint32)
    step = np.broadcast_to((d * (2 * s.astype(np.float32) + 1) / 8.0)[..., None], wb.shape)
    idx = _nearest_grid(_safe_div(np.abs(wb), step).reshape(n * 32, 8), grid).reshape(n, 32).astype(np.uint32)
    w8 = w.reshape(n * 32, 8)
    if wtype == F.IQ2_S:
        neg = w8 < 0
        signs = np.zeros(n * 32, np.uint8)
        for j in range(8):
            signs |= neg[:, j].astype(np.uint8) << j
        signs = signs.reshape(n, 32)
        qh = np.zeros((n, 8), np.uint8)
        for l in range(4):
            qh |= ((idx[:, l::4] >> 8) & 3).astype(np.uint8) << (2 * l)
        sc = (s[:, 0::2] | (s[:, 1::2] << 4)).astype(np.uint8)
        return np.concatenate([dbytes.reshape(n, 2), (idx & 0xFF).astype(np.uint8), signs, qh, sc], axis=1)
    signs = (_even_signs(w8) & 0x7F).astype(np.uint32).reshape(n, 32)
    if wtype == F.IQ2_XS:
        qs = (idx | (signs << 9)).astype("<u2").view(np.uint8).reshape(n, 64)
        sc = (s[:, 0::2] | (s[:, 1::2] << 4)).astype(np.uint8)
        return np.concatenate([dbytes.reshape(n, 2), qs, sc], axis=1)
    i4, s4 = idx.reshape(n, 8, 4), signs.reshape(n, 8, 4)
    lo = i4[..., 0] | (i4[..., 1] << 8) | (i4[..., 2] << 16) | (i4[..., 3] << 24)
    hi = s4[..., 0] | (s4[..., 1] << 7) | (s4[..., 2] << 14) | (s4[..., 3] << 21) | (s << 28)
    qs = np.stack([lo, hi], axis=-1).astype("<u4").view(np.uint8).reshape(n, 64)
    return np.concatenate([dbytes.reshape(n, 2), qs], axis=1)


def _enc_iq1_m(w):
    """qs[32] | qh[16] | scales[8]: weight = d (2 s + 1) (g + delta), g in {-1, 0, 1}^8 from a 2048-entry grid, delta = +-1/8
    per group of eight, a 3-bit scale per 16 weights, the fp16 d spread over the top nibbles of the scale halfwords."""
    from gguf.quants import IQ1_M

    IQ1_M.init_grid()
    grid = IQ1_M.grid.reshape(2048, 8).astype(np.float32)
    n = w.shape[0]
    wb = w.reshape(n, 16, 16)
    step_t = np.abs(wb).max(-1) / 1.125
    d, dbytes = _f16(step_t.max(-1, keepdims=True) / 15.0)
    s = np.clip(np.rint((_safe_div(step_t, d) - 1.0) / 2.0), 0, 7).astype(np.uint32)
    step = np.broadcast_to((d * (2 * s.astype(np.float32) + 1))[..., None], wb.shape)
    v = _safe_div(wb, step).reshape(n * 32, 8)
    ip, im = _nearest_grid(v - 0.125, grid), _nearest_grid(v + 0.125, grid)
    ep, em = ((grid[ip] + 0.125 - v) ** 2).sum(-1), ((grid[im] - 0.125 - v) ** 2).sum(-1)
    neg = em < ep
    idx = np.where(neg, im, ip).astype(np.uint32).reshape(n, 32)
    nib = ((idx >> 8) & 7) | (neg.reshape(n, 32).astype(np.uint32) << 3)
    qh = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    dbits = dbytes.reshape(n, 2).astype(np.uint32)
    dv = dbits[:, 0] | (dbits[:, 1] << 8)
    s4 = s.reshape(n, 4, 4)
    sc = (s4[..., 0] | (s4[..., 1] << 3) | (s4[..., 2] << 6) | (s4[..., 3] << 9)).astype(np.uint32)
    for i in range(4):
        sc[:, i] |= ((dv >> (4 * i)) & 0xF) << 12
    return np.concatenate([(idx & 0xFF).astype(np.uint8), qh, sc.astype("<u2").view(np.uint8).reshape(n, 8)], axis=1)


def _enc_gguf(wtype):
    def enc(w):
        from gguf.constants import GGMLQuantizationType
        from gguf.quants import quantize

        return quantize(np.ascontiguousarray(w.reshape(-1, 32)), GGMLQuantizationType(wtype)).reshape(w.shape[0], -1)
    return enc


_ENCODERS = {F.Q4_K: _enc_q4_k, F.Q5_K: _enc_q5_k, F.Q2_K: _enc_q2_k, F.Q3_K: _enc_q3_k, F.Q6_K: _enc_q6_k,
             F.IQ4_NL: _enc_iq4_nl, F.IQ4_XS: _enc_iq4_xs, F.IQ3_S: _enc_iq3_s, F.IQ3_XXS: _enc_iq3_xxs,
             F.IQ2_XXS: lambda w: _enc_iq2(w, F.IQ2_XXS), F.IQ2_XS: lambda w: _enc_iq2(w, F.IQ2_XS), F.IQ2_S: lambda w: _enc_iq2(w, F.IQ2_S), F.IQ1_M: _enc_iq1_m,
             F.Q8_0: _enc_gguf(F.Q8_0), F.Q4_0: _enc_gguf(F.Q4_0), F.Q5_0: _enc_gguf(F.Q5_0)}


def encode(w: np.ndarray, wtype: int) -> np.ndarray:
    """fp32 [n_out, K] -> raw GGUF block bytes uint8 [n_out, (K/256) * bytes_per_256] of the type."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n_out, k = w.shape
    if k % F.QK:
        raise ValueError(f"K={k} is not a multiple of {F.QK}")
    nb = k // F.QK
    out = np.empty((n_out, nb, F.BYTES_PER_256[wtype]), np.uint8)
    enc = _ENCODERS[wtype]
    step = max(1, 65536 // nb)
    for r0 in range(0, n_out, step):
        blk = w[r0:r0 + step].reshape(-1, F.QK)
        out[r0:r0 + step] = enc(blk).reshape(-1, nb, F.BYTES_PER_256[wtype])
    return out.reshape(n_out, -1)


def encoded_weights(n_out: int, k: int, wtype: int, seed: int, sigma: float = 0.02) -> np.ndarray:
    return encode(gaussian_weights(n_out, k, seed, sigma), wtype)
