"""GGUF block-quant dequantisation (Q4_0, Q8_0, Q3_K, Q4_K, Q5_K, Q6_K): the vectorised loader
against scalar restatements of the block formats, on random block bytes.

Reference: src/vllm/model_executor/model_loader/gguf_dequant.cpp, src/vt/cpu/cpu_quant_dequant.cpp
(the same ggml block layouts)."""
import struct

import numpy as np
import pytest

from vllm_cpp_b200.loader import gguf

RNG = np.random.default_rng(11)


def f16(b: bytes) -> float:
    return float(np.frombuffer(b, dtype=np.float16)[0])


def rand_block(nbytes: int, f16_at) -> bytes:
    """Random bytes with finite, small fp16 scales at the given offsets."""
    raw = bytearray(RNG.integers(0, 256, nbytes, dtype=np.uint8).tobytes())
    for off in f16_at:
        raw[off:off + 2] = np.float16(RNG.uniform(-0.5, 0.5)).tobytes()
    return bytes(raw)


def scale_min_k4(j, q):
    if j < 4:
        return q[j] & 63, q[j + 4] & 63
    return (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4), (q[j + 4] >> 4) | ((q[j] >> 6) << 4)


def scalar_q4_0(b):
    d = f16(b[0:2])
    qs = b[2:18]
    return [((qs[j] & 0xF) - 8) * d for j in range(16)] + [((qs[j] >> 4) - 8) * d for j in range(16)]


def scalar_q8_0(b):
    d = f16(b[0:2])
    return [struct.unpack("b", b[2 + j:3 + j])[0] * d for j in range(32)]


def scalar_q4_k(b):
    d, dmin = f16(b[0:2]), f16(b[2:4])
    sc, q = b[4:16], b[16:144]
    y, isx = [], 0
    for j in range(4):
        s1, m1 = scale_min_k4(isx, sc)
        s2, m2 = scale_min_k4(isx + 1, sc)
        blk = q[32 * j:32 * j + 32]
        y += [d * s1 * (x & 0xF) - dmin * m1 for x in blk]
        y += [d * s2 * (x >> 4) - dmin * m2 for x in blk]
        isx += 2
    return y


def scalar_q5_k(b):
    d, dmin = f16(b[0:2]), f16(b[2:4])
    sc, qh, ql = b[4:16], b[16:48], b[48:176]
    y, isx, u1, u2 = [], 0, 1, 2
    for j in range(4):
        s1, m1 = scale_min_k4(isx, sc)
        s2, m2 = scale_min_k4(isx + 1, sc)
        blk = ql[32 * j:32 * j + 32]
        y += [d * s1 * ((blk[l] & 0xF) + (16 if qh[l] & u1 else 0)) - dmin * m1 for l in range(32)]
        y += [d * s2 * ((blk[l] >> 4) + (16 if qh[l] & u2 else 0)) - dmin * m2 for l in range(32)]
        isx += 2
        u1 <<= 2
        u2 <<= 2
    return y


def scalar_q6_k(b):
    ql, qh = b[0:128], b[128:192]
    sc = [struct.unpack("b", b[192 + i:193 + i])[0] for i in range(16)]
    d = f16(b[208:210])
    y = [0.0] * 256
    for n in range(2):
        L, H, S = ql[64 * n:64 * n + 64], qh[32 * n:32 * n + 32], sc[8 * n:8 * n + 8]
        for l in range(32):
            i = l // 16
            q1 = ((L[l] & 0xF) | (((H[l] >> 0) & 3) << 4)) - 32
            q2 = ((L[l + 32] & 0xF) | (((H[l] >> 2) & 3) << 4)) - 32
            q3 = ((L[l] >> 4) | (((H[l] >> 4) & 3) << 4)) - 32
            q4 = ((L[l + 32] >> 4) | (((H[l] >> 6) & 3) << 4)) - 32
            y[128 * n + l] = d * S[i] * q1
            y[128 * n + l + 32] = d * S[i + 2] * q2
            y[128 * n + l + 64] = d * S[i + 4] * q3
            y[128 * n + l + 96] = d * S[i + 6] * q4
    return y


def scalar_q3_k(b):
    hm, qs, scr = b[0:32], b[32:96], b[96:108]
    d = f16(b[108:110])
    aux = list(struct.unpack("<III", scr)) + [0]
    k1, k2 = 0x03030303, 0x0F0F0F0F
    tmp = aux[2]
    aux[2] = ((aux[0] >> 4) & k2) | (((tmp >> 4) & k1) << 4)
    aux[3] = ((aux[1] >> 4) & k2) | (((tmp >> 6) & k1) << 4)
    aux[0] = (aux[0] & k2) | (((tmp >> 0) & k1) << 4)
    aux[1] = (aux[1] & k2) | (((tmp >> 2) & k1) << 4)
    scales = [s - 32 for s in struct.unpack("16b", struct.pack("<IIII", *aux))]
    y, isx, m = [], 0, 1
    for n in range(2):
        q = qs[32 * n:32 * n + 32]
        shift = 0
        for _ in range(4):
            for part in range(2):
                dl = d * scales[isx]
                isx += 1
                for l in range(16):
                    x = q[16 * part + l]
                    y.append(dl * (((x >> shift) & 3) - (0 if hm[16 * part + l] & m else 4)))
            shift += 2
            m <<= 1
    return y


CASES = {
    2: (scalar_q4_0, [0]),
    8: (scalar_q8_0, [0]),
    11: (scalar_q3_k, [108]),
    12: (scalar_q4_k, [0, 2]),
    13: (scalar_q5_k, [0, 2]),
    14: (scalar_q6_k, [208]),
}


@pytest.mark.parametrize("ggml_type", sorted(CASES))
def test_block_dequant_matches_scalar_restatement(ggml_type):
    name, per_block, nbytes = gguf.GGML[ggml_type]
    scalar, f16_at = CASES[ggml_type]
    blocks = [rand_block(nbytes, f16_at) for _ in range(3)]
    want = np.array([v for b in blocks for v in scalar(b)], dtype=np.float64).reshape(3, per_block)
    raw = np.frombuffer(b"".join(blocks), dtype=np.uint8)
    got = gguf.dequantize(raw, ggml_type, (3, per_block)).astype(np.float64)
    assert got.shape == want.shape
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6, err_msg=name)
