"""CPU check of the index arithmetic of the any-precision lookup decoder (`csrc/gemv_anyprec_pipe.cuh`:
`ap_fields`, `ap_lookup_word`), restated in Python with the same shifts and masks, against the oracle's packer of the
reference layout (`decdec_extension/anyprec.cu:261-331`: bit 31-8j-r of word t of a block holds channel
block_start + 8*E*j + 8*t + r, plane 0 is the most significant code bit).  The kernel itself is compared with the oracle
on the GPU (`tests/test_gpu_parity.py::test_anyprec_gemv`); this test pins the regrouping where no GPU is present."""
import numpy as np
import pytest

from oracle import formats

M32 = 0xFFFFFFFF


def _rotr(v, i):
    i %= 32
    return ((v >> i) | (v << (32 - i))) & M32 if i else v


def _rotl(v, i):
    i %= 32
    return ((v << i) | (v >> (32 - i))) & M32 if i else v


def fields(planes):
    """ap_fields<B>: field t of result ph = bits of planes 0..B-1 (most significant first) at position 4t + ph."""
    B = len(planes)
    rot = [_rotr(planes[i], i) for i in range(B)]
    out = []
    for ph in range(4):
        m = 0
        for i in range(B):
            m |= rot[i] & ((0x11111111 << ((ph - i) & 3)) & M32)
        out.append(_rotl(m, (B - 1 - ph) & 31))
    return out


def word_codes(q, bits):
    """ap_lookup_word: {(j, r): code} for the 32 channels of one plane-word position, from the byte offsets the kernel forms."""
    bh = min(bits, 4)
    bl = bits - bh
    vh = fields(q[:bh])
    vl = fields(q[4:4 + bl]) if bl else [0] * 4
    codes = {}
    for ph in range(4):
        for t in range(8):
            pos = 31 - (4 * t + ph)
            j, r = pos >> 3, pos & 7
            if bl == 0:
                off = ((vh[ph] >> (4 * t - 1)) & 0x1E) if t else ((vh[ph] << 1) & 0x1E)
            else:
                mh, ml = 0xF << (bl + 1), ((1 << bl) - 1) << 1
                sh = 4 * t - bl - 1
                off = ((vh[ph] >> sh) if sh >= 0 else (vh[ph] << -sh)) & mh
                off |= ((vl[ph] >> (4 * t - 1)) if t else (vl[ph] << 1)) & ml
            assert off % 2 == 0 and off < (2 << bits)
            codes[(j, r)] = off >> 1
    return codes


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("K", [128, 1024, 1536])
def test_lookup_offsets_recover_the_packed_codes(bits, K):
    rng = np.random.default_rng(bits * 100 + K)
    N = 2
    want = rng.integers(0, 2 ** bits, size=(N, K)).astype(np.int32)
    qw = formats.anyprec_pack(want, bits).view(np.uint32)            # [bits, N, K/32]
    nwords = K // 32
    nfull, tail = nwords >> 5, nwords & 31
    for n in range(N):
        for wi in range(nwords):
            blk, t = wi >> 5, wi & 31
            E = tail if blk == nfull else 32
            got = word_codes([int(qw[pl, n, wi]) for pl in range(bits)], bits)
            assert len(got) == 32
            for (j, r), c in got.items():
                assert c == want[n, blk * 1024 + 8 * E * j + 8 * t + r]
