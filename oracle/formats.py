"""Weight formats of the base GEMV: quantizers, packers and dequantizers (CPU oracle, numpy).

Test infrastructure only.  Every function names the reference source it restates
(paths are relative to the SNU-ARC/DecDEC repository).
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------------------------
# AWQ-style asymmetric uniform quantization and its binary-coded (LUT-GEMM) form
# ----------------------------------------------------------------------------------------------


def pseudo_quantize_uniform(w: np.ndarray, n_bit: int, group: int):
    """Asymmetric per-group uniform quantizer.

    Follows `decdec_setup/llm-awq/quantize/quantizer.py:216-258` (zero_point=True branch), in
    float32 like the reference when it is fed float32 weights.

    w: [N, K] float.  Returns (w_fake [N,K] f32, scales [N,K/group] f32, zeros [N,K/group] f32,
    codes [N,K] int32 in [0, 2^n_bit - 1]).
    """
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % group == 0
    g = w.reshape(-1, group)
    max_val = g.max(axis=1, keepdims=True)
    min_val = g.min(axis=1, keepdims=True)
    max_int = np.float32(2 ** n_bit - 1)
    scales = np.maximum(max_val - min_val, np.float32(1e-5)) / max_int
    zeros = np.clip(-np.rint(min_val / scales), 0, max_int).astype(np.float32)
    codes = np.clip(np.rint(g / scales) + zeros, 0, max_int).astype(np.float32)
    w_fake = ((codes - zeros) * scales).astype(np.float32)
    return (
        w_fake.reshape(n, k),
        scales.reshape(n, k // group),
        zeros.reshape(n, k // group),
        codes.reshape(n, k).astype(np.int32),
    )


def uniform_to_bcq(scales: np.ndarray, zeros: np.ndarray, codes: np.ndarray, n_bit: int):
    """Uniform codes -> binary-coded tensors of the LUT-GEMM kernel.

    Follows `decdec_setup/llm-awq/quantize/qmodule.py:61-92` (`convert_bcq_format`):
    alpha_p = scale * 2^p / 2, q_bias = sum_p alpha_p - scale * zero, plane p = bit p of the code,
    bit j of word kw holds input channel 32*kw + j.

    scales, zeros: [N, G] float32, codes: [N, K] int.  Returns
    (qweight int32 [K/32, n_bit, N], alpha f32 [G, n_bit, N], q_bias f32 [G, N]).
    """
    scales = np.asarray(scales, np.float32)
    zeros = np.asarray(zeros, np.float32)
    n, k = codes.shape
    pw = np.array([2 ** i for i in range(n_bit)], np.float32)
    alpha = (scales / np.float32(2.0))[:, :, None] * pw[None, None, :]  # [N, G, B]
    offset = alpha.sum(-1) - scales * zeros  # [N, G]
    bits = ((codes[:, :, None].astype(np.int64) >> np.arange(n_bit)) & 1)  # [N, K, B]
    bits = bits.transpose(0, 2, 1).reshape(n, n_bit, k // 32, 32)  # [N, B, K/32, 32]
    words = (bits.astype(np.uint64) << np.arange(32, dtype=np.uint64)).sum(-1).astype(np.uint32)
    qweight = words.transpose(2, 1, 0).copy().view(np.int32)  # [K/32, B, N]
    return qweight, alpha.transpose(1, 2, 0).copy(), offset.transpose(1, 0).copy()


def bcq_dequant(qweight: np.ndarray, alpha: np.ndarray, q_bias: np.ndarray, group: int,
                dtype=np.float64) -> np.ndarray:
    """Dense [N, K] weights of a binary-coded layer.

    Follows `evaluation/evaltools.py:546-580` (`lutgemm_dequant`), but evaluates the sum in `dtype`
    (float64 by default) instead of fp16, so it is the exact value of the stored tensors:
    W[n,k] = sum_p alpha[g(k),p,n] * (2*bit_p(k,n) - 1) + q_bias[g(k),n].
    """
    kw, b, n = qweight.shape
    k = kw * 32
    words = qweight.view(np.uint32)
    bits = (words[:, :, :, None] >> np.arange(32, dtype=np.uint32)) & 1  # [KW, B, N, 32]
    bits = bits.transpose(0, 3, 1, 2).reshape(k, b, n)
    delta = bits.astype(dtype) * 2 - 1
    gidx = np.arange(k) // group
    w = (delta * alpha.astype(dtype)[gidx]).sum(1) + q_bias.astype(dtype)[gidx]
    return w.T.copy()  # [N, K]


# ----------------------------------------------------------------------------------------------
# Non-uniform (per-output-row LUT) quantization: any-precision and SqueezeLLM containers
# ----------------------------------------------------------------------------------------------


def lut_quantize(w: np.ndarray, n_bit: int, iters: int = 4):
    """Seeded-free, deterministic "k-means-like" per-row centroids (stand-in for the SqueezeLLM
    quantizer of the un-vendored `decdec_setup/any-precision-llm` submodule).

    Centroids start at row quantiles and take a few Lloyd iterations.  Returns
    (lut fp16 [N, 2^n_bit] ascending, codes int32 [N, K]) with codes = nearest fp16 centroid.
    """
    w = np.asarray(w, np.float32)
    n, k = w.shape
    c = 2 ** n_bit
    qs = (np.arange(c, dtype=np.float32) + 0.5) / c
    cent = np.quantile(w, qs, axis=1).T.astype(np.float32)  # [N, C]
    for _ in range(iters):
        codes = np.abs(w[:, :, None] - cent[:, None, :]).argmin(-1)
        for j in range(c):
            m = codes == j
            cnt = m.sum(1)
            s = (w * m).sum(1)
            cent[:, j] = np.where(cnt > 0, s / np.maximum(cnt, 1), cent[:, j])
        cent.sort(axis=1)
    lut = np.ascontiguousarray(cent).astype(np.float16)
    codes = np.abs(w[:, :, None] - lut.astype(np.float32)[:, None, :]).argmin(-1).astype(np.int32)
    return lut, codes


def lut_dequant(lut: np.ndarray, codes: np.ndarray, dtype=np.float64) -> np.ndarray:
    """W[n,k] = lut[n, codes[n,k]]; follows `decdec_setup/conv_sqllm.py:76-87`."""
    return np.take_along_axis(lut.astype(dtype), codes.astype(np.int64), axis=1)


def anyprec_k_of(K: int):
    """Input-channel index held by (word, bit) of one any-precision bit-plane row.

    Derived from the store pattern of `decdec_extension/anyprec.cu:261-331`
    (`dequant_kbit_store`): a row is cut into blocks of 1024 channels (32 words); inside a block of
    E words (E = 32, or (K mod 1024)/32 for the tail block) bit 31-8j-r of word t holds channel
    block_start + 8*E*j + 8*t + r   (j in 0..3, r in 0..7).
    Returns int array kmap[K/32, 32] indexed [word, bit].
    """
    assert K % 32 == 0
    nw = K // 32
    kmap = np.zeros((nw, 32), np.int64)
    for i in range((nw + 31) // 32):
        e = min(32, nw - 32 * i)
        for t in range(e):
            for j in range(4):
                for r in range(8):
                    kmap[32 * i + t, 31 - 8 * j - r] = 1024 * i + 8 * e * j + 8 * t + r
    return kmap


def anyprec_pack(codes: np.ndarray, n_bit: int) -> np.ndarray:
    """codes [N, K] (0..2^n_bit-1) -> bit-plane tensor int32 [n_bit, N, K/32]; plane 0 is the most
    significant bit of the code (`decdec_extension/anyprec.cu:24-27`: q[0] lands on the highest
    nibble bit)."""
    n, k = codes.shape
    kmap = anyprec_k_of(k)  # [W, 32]
    g = codes[:, kmap]  # [N, W, 32]
    out = np.zeros((n_bit, n, k // 32), np.uint32)
    sh = np.arange(32, dtype=np.uint64)
    for p in range(n_bit):
        bit = (g >> (n_bit - 1 - p)) & 1
        out[p] = (bit.astype(np.uint64) << sh).sum(-1).astype(np.uint32)
    return out.view(np.int32)


def anyprec_unpack(qweight: np.ndarray, n_bit: int) -> np.ndarray:
    """Inverse of `anyprec_pack`; uses only the first n_bit planes (the reference accepts tensors
    with more planes than `bitwidth`, `decdec_extension/decdec.cu:295`)."""
    _, n, nw = qweight.shape
    k = nw * 32
    kmap = anyprec_k_of(k)
    words = qweight.view(np.uint32)
    codes = np.zeros((n, k), np.int32)
    for p in range(n_bit):
        bits = ((words[p][:, :, None] >> np.arange(32, dtype=np.uint32)) & 1).astype(np.int32)
        tmp = np.zeros((n, k), np.int32)
        tmp[:, kmap.reshape(-1)] = bits.reshape(n, -1)
        codes |= tmp << (n_bit - 1 - p)
    return codes


def anyprec_reference_emulation_3bit(qweight: np.ndarray, lut: np.ndarray) -> np.ndarray:
    """Literal numpy emulation of the 3-bit path of `dequant_kbit_store`
    (`decdec_extension/anyprec.cu:38-66` bit transposition, `:310-329` lookup and store order) for
    K a multiple of 32.  Used only to pin `anyprec_k_of`/`anyprec_pack` to the reference layout."""
    _, n, nw = qweight.shape
    k = nw * 32
    q = qweight.view(np.uint32).astype(np.uint64)
    out = np.zeros((n, k), lut.dtype)
    m0, m1, m2, m3 = 0x88888888, 0x44444444, 0x22222222, 0x11111111
    mask = 0x0F0F0F0F
    for i in range((nw + 31) // 32):
        eff = min(32, nw - 32 * i)
        for t in range(eff):
            a, b, c = q[0, :, 32 * i + t], q[1, :, 32 * i + t], q[2, :, 32 * i + t]
            qw = [None] * 8
            qw[0] = ((a & m0) | ((b & m0) >> 1) | ((c & m0) >> 2)) >> 1
            qw[1] = (a & m1) | ((b & m1) >> 1) | ((c & m1) >> 2)
            qw[2] = ((a & m2) << 1) | (b & m2) | ((c & m2) >> 1)
            qw[3] = ((a & m3) << 2) | ((b & m3) << 1) | (c & m3)
            for z in range(4):
                qw[4 + z] = qw[z] & mask
            for z in range(4):
                qw[z] = (qw[z] >> 4) & mask
            dq = np.zeros((n, 16, 2), lut.dtype)
            for j in range(3, -1, -1):
                for kk in range(4):
                    x = np.take_along_axis(lut, (qw[kk * 2 + 0] & 0xFF).astype(np.int64)[:, None], 1)[:, 0]
                    y = np.take_along_axis(lut, (qw[kk * 2 + 1] & 0xFF).astype(np.int64)[:, None], 1)[:, 0]
                    dq[:, j * 4 + kk, 0] = x
                    dq[:, j * 4 + kk, 1] = y
                for z in range(8):
                    qw[z] = qw[z] >> 8
            for j in range(4):
                base = 8 * eff * j + i * 1024 + 8 * t
                out[:, base:base + 8] = dq[:, 4 * j:4 * j + 4, :].reshape(n, 8)
    return out


def sqllm_pack(codes: np.ndarray, n_bit: int) -> np.ndarray:
    """codes [N, K] -> SqueezeLLM dense packing int32 [K*n_bit/32, N].

    Inverse of `evaluation/evaltools.py:583-645` (`sqllm_dequant`) and of the decode order of
    `decdec_extension/sqllm.cu:64-113,155-162`: 4-bit packs 8 consecutive channels per word at bit
    4*i; 3-bit packs 32 consecutive channels into a 96-bit little-endian string over 3 words.
    """
    n, k = codes.shape
    c = codes.astype(np.uint64)
    if n_bit == 4:
        g = c.reshape(n, k // 8, 8)
        words = (g << (4 * np.arange(8, dtype=np.uint64))).sum(-1).astype(np.uint32)
        return words.T.copy().view(np.int32)
    assert n_bit == 3 and k % 32 == 0
    g = c.reshape(n, k // 32, 32)
    words = np.zeros((n, k // 32, 3), np.uint64)
    for i in range(32):
        pos = 3 * i
        wi, off = pos // 32, pos % 32
        words[:, :, wi] |= (g[:, :, i] << np.uint64(off)) & np.uint64(0xFFFFFFFF)
        if off > 29:
            words[:, :, wi + 1] |= g[:, :, i] >> np.uint64(32 - off)
    return words.reshape(n, -1).astype(np.uint32).T.copy().view(np.int32)


def sqllm_unpack(qweight: np.ndarray, n_bit: int) -> np.ndarray:
    """Packed SqueezeLLM tensor [K*n_bit/32, N] -> codes [N, K]; follows
    `evaluation/evaltools.py:583-645`."""
    w = qweight.view(np.uint32).T.astype(np.uint64)  # [N, words]
    n = w.shape[0]
    if n_bit == 4:
        codes = (w[:, :, None] >> (4 * np.arange(8, dtype=np.uint64))) & 0xF
        return codes.reshape(n, -1).astype(np.int32)
    assert n_bit == 3
    g = w.reshape(n, -1, 3)
    codes = np.zeros((n, g.shape[1], 32), np.int32)
    # 96-bit little-endian string: bits 0..63 live in `lo`, bits 64..95 in `hi`
    lo = g[:, :, 0] | (g[:, :, 1] << np.uint64(32))
    hi = g[:, :, 2]
    for i in range(32):
        pos = 3 * i
        if pos + 3 <= 64:
            v = (lo >> np.uint64(pos)) & 7
        elif pos >= 64:
            v = (hi >> np.uint64(pos - 64)) & 7
        else:  # straddles bit 64
            v = ((lo >> np.uint64(pos)) | (hi << np.uint64(64 - pos))) & 7
        codes[:, :, i] = v.astype(np.int32)
    return codes.reshape(n, -1)
