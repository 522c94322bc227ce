"""Bucket-threshold top-k channel selection (CPU oracle of `decdec_extension/dec.cu:78-182`).

Test infrastructure only.  The reference has no CPU implementation of this step; this file restates
the CUDA kernel's arithmetic exactly (including the mixed half/float recipe of the bucket bounds)
and fixes what the kernel leaves to chance: the reference appends rows to a bucket in atomic-arrival
order (`dec.cu:146-154`), so which members of the overflowing bucket are taken, and the order of the
published rows, vary from run to run; here the lowest channel indices are taken and the order is fixed.
"""
from __future__ import annotations

import numpy as np

CHUNK = 1024        # `decdec_extension/macros.h:8`
NUM_BUCKETS = 32    # `decdec_extension/macros.h:18`


def _round_bf16(v: float) -> float:
    """Round a Python float to the nearest bfloat16 (ties to even), without double rounding."""
    if v == 0.0 or not np.isfinite(v):
        return float(v)
    m, e = np.frexp(v)            # v = m * 2**e, 0.5 <= |m| < 1
    q = np.rint(m * 256.0)        # 8 significant bits
    return float(np.ldexp(q, e - 8))


def _rn(v: float, dtype: str) -> float:
    """Round a double to the activation dtype (one correctly rounded step)."""
    if dtype == "fp16":
        return float(np.float16(np.float64(v)))
    if dtype == "bf16":
        return _round_bf16(float(v))
    if dtype == "fp32":
        return float(np.float32(np.float64(v)))
    raise ValueError(dtype)


def bucket_floors(a: float, b: float, dtype: str) -> np.ndarray:
    """Lower bounds of the 32 buckets, as float64 holding exactly the dtype values.

    Follows `decdec_extension/dec.cu:117-130`:
      L < 16 : floor = a + DT( float(DT(b - a)) * L / 15 )       (DT subtract, float mul, float div,
                                                                  round to DT, DT add)
      L >= 16: floor = DT( float(b) * (31 - L) / 16 )
    a and b are values of the activation dtype (thresholds[0] and thresholds[k-1],
    `decdec_extension/decdec.cu:66-67`).
    """
    a = _rn(a, dtype)
    b = _rn(b, dtype)
    floors = np.zeros(NUM_BUCKETS, np.float64)
    diff = _rn(np.float64(b) - np.float64(a), dtype)          # DT subtract (exact in double, one rounding)
    for L in range(NUM_BUCKETS):
        if L < 16:
            t = np.float32(np.float32(diff) * np.float32(L))  # float multiply
            t = np.float32(t / np.float32(15))                # float divide
            floors[L] = _rn(np.float64(a) + np.float64(_rn(float(t), dtype)), dtype)
        else:
            t = np.float32(np.float32(b) * np.float32(31 - L))
            t = np.float32(t / np.float32(16))
            floors[L] = _rn(float(t), dtype)
    return floors


def select(x: np.ndarray, a: float, b: float, k_chunk: int, dtype: str = "fp16"):
    """Channel selection for one activation vector.

    x: [K] values of the activation dtype (any float array holding them exactly).
    Returns (rows int32 [k], acts float64 [k], hist int64 [num_chunks, 32]) where
    k = k_chunk*K // 1024 (`dec.cu:48`), the picks of chunk c sit at rows[c*k_chunk : c*k_chunk+kq]
    (`dec.cu:169-170`), and hist[c, L] is the population of bucket L in chunk c.

    Per chunk c of length len <= 1024: kq = k_chunk*len // 1024 (`dec.cu:84-86`).  Bucket L holds the
    channels with floor[L] <= |x| < ceil[L], ceil[0] = +inf, ceil[L] = floor[L-1]
    (`dec.cu:133-137,145`); for floors that do not increase with L this is the LOWEST L with
    floor[L] <= |x|, which is how the bucket is computed here (NaN and inf fall in no bucket).
    Buckets are drained in order 0,1,2,... until kq rows are taken (`dec.cu:161-177`).

    What the reference leaves to chance, and this oracle fixes:
      * which members of the bucket that overflows the quota are taken (reference: atomic arrival
        order, `dec.cu:146-154`; here: the lowest channel indices);
      * the order of the published rows (here: members of the fully taken buckets by ascending
        channel index, then the picks of the overflowing bucket by ascending channel index).
    Degenerate thresholds (floor[16] > floor[15], which needs thresholds[0] > ~1000*thresholds[k-1]
    in fp16) could make the reference count one channel in two buckets; here it is in the lower one.
    If a chunk has fewer than kq finite channels the reference trips a device assert (`dec.cu:178`);
    the oracle (and the CUDA library) pad with (first channel of the chunk, activation 0).
    """
    x = np.asarray(x, np.float64).reshape(-1)
    K = x.shape[0]
    k_total = k_chunk * K // CHUNK
    floors = bucket_floors(a, b, dtype)
    num_chunks = (K + CHUNK - 1) // CHUNK
    rows = np.zeros(k_total, np.int32)
    acts = np.zeros(k_total, np.float64)
    hist = np.zeros((num_chunks, NUM_BUCKETS), np.int64)
    for c in range(num_chunks):
        s, e = c * CHUNK, min((c + 1) * CHUNK, K)
        kq = k_chunk * (e - s) // CHUNK
        ax = np.abs(x[s:e])
        with np.errstate(invalid="ignore"):
            ge = ax[:, None] >= floors[None, :]                      # [len, 32]
        bucket = np.where(ge.any(1) & np.isfinite(ax), ge.argmax(1), NUM_BUCKETS)
        hist[c] = np.bincount(bucket, minlength=NUM_BUCKETS + 1)[:NUM_BUCKETS]
        cum = np.cumsum(hist[c])
        over = np.nonzero(cum >= kq)[0]
        lb = int(over[0]) if over.size else NUM_BUCKETS
        full = np.nonzero(bucket < lb)[0]                            # ascending index
        taken = list(s + full)
        if lb < NUM_BUCKETS:
            quota = kq - len(taken)
            taken.extend((s + np.nonzero(bucket == lb)[0][:quota]).tolist())
        for i in range(kq):
            pos = c * k_chunk + i
            if i < len(taken):
                rows[pos] = taken[i]
                acts[pos] = x[taken[i]]
            else:
                rows[pos] = s
                acts[pos] = 0.0
    return rows, acts, hist


def exact_topk(x: np.ndarray, k: int) -> np.ndarray:
    """Exact global top-k of |x| (`evaluation/evaltools.py:336`), the index set that
    `unfused_dec` is fed by the evaluation harness."""
    ax = np.abs(np.asarray(x, np.float64).reshape(-1))
    return np.argsort(-ax, kind="stable")[:k].astype(np.int32)
