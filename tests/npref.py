"""Independent numpy statement of the GGUF block formats, written from the format
definition (not from the oracle's C code) so the two can be checked against each other."""
import numpy as np


def f16(b):
    return np.frombuffer(bytes(b), dtype=np.float16).astype(np.float32)


def deq_q4_0(data):
    blocks = np.asarray(data, dtype=np.uint8).reshape(-1, 18)
    d = blocks[:, 0:2].copy().view(np.float16).astype(np.float32)  # [nb,1]
    q = blocks[:, 2:]
    lo = (q & 15).astype(np.int32) - 8
    hi = (q >> 4).astype(np.int32) - 8
    return (d * np.concatenate([lo, hi], axis=1).astype(np.float32)).reshape(-1)


def deq_q8_0(data):
    blocks = np.asarray(data, dtype=np.uint8).reshape(-1, 34)
    d = blocks[:, 0:2].copy().view(np.float16).astype(np.float32)
    return (d * blocks[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)


def q4k_scales(sc12):
    """12 packed bytes -> (8 scales, 8 mins), 6 bits each."""
    s = [int(x) for x in sc12]
    sc, mn = [], []
    for j in range(8):
        if j < 4:
            sc.append(s[j] & 63)
            mn.append(s[j + 4] & 63)
        else:
            sc.append((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4))
            mn.append((s[j + 4] >> 4) | ((s[j] >> 6) << 4))
    return sc, mn


def pack_q4k_scales(sc, mn):
    """Inverse of q4k_scales."""
    out = [0] * 12
    for j in range(4):
        out[j] = (sc[j] & 63) | ((sc[j + 4] >> 4) << 6)
        out[j + 4] = (mn[j] & 63) | ((mn[j + 4] >> 4) << 6)
        out[j + 8] = (sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4)
    return out


def deq_q4_k(data):
    blocks = np.asarray(data, dtype=np.uint8).reshape(-1, 144)
    out = np.empty((blocks.shape[0], 256), dtype=np.float32)
    for b, blk in enumerate(blocks):
        d = np.float32(f16(blk[0:2])[0])
        dmin = np.float32(f16(blk[2:4])[0])
        sc, mn = q4k_scales(blk[4:16])
        qs = blk[16:]
        for g in range(4):
            q = qs[32 * g:32 * g + 32]
            d1 = np.float32(d * np.float32(sc[2 * g]))
            m1 = np.float32(dmin * np.float32(mn[2 * g]))
            d2 = np.float32(d * np.float32(sc[2 * g + 1]))
            m2 = np.float32(dmin * np.float32(mn[2 * g + 1]))
            out[b, 64 * g:64 * g + 32] = d1 * (q & 15).astype(np.float32) - m1
            out[b, 64 * g + 32:64 * g + 64] = d2 * (q >> 4).astype(np.float32) - m2
    return out.reshape(-1)


def deq_q6_k(data):
    blocks = np.asarray(data, dtype=np.uint8).reshape(-1, 210)
    out = np.empty((blocks.shape[0], 256), dtype=np.float32)
    for b, blk in enumerate(blocks):
        ql, qh, sc = blk[0:128], blk[128:192], blk[192:208].view(np.int8)
        d = np.float32(f16(blk[208:210])[0])
        for c in range(2):
            for l in range(32):
                isx = l // 16
                lo, hi, h = int(ql[64 * c + l]), int(ql[64 * c + l + 32]), int(qh[32 * c + l])
                qv = [(lo & 15) | ((h & 3) << 4), (hi & 15) | (((h >> 2) & 3) << 4),
                      (lo >> 4) | (((h >> 4) & 3) << 4), (hi >> 4) | (((h >> 6) & 3) << 4)]
                for j in range(4):
                    s = np.float32(sc[8 * c + isx + 2 * j])
                    out[b, 128 * c + l + 32 * j] = np.float32(d * s) * np.float32(qv[j] - 32)
    return out.reshape(-1)


DEQ = {2: deq_q4_0, 8: deq_q8_0, 12: deq_q4_k, 14: deq_q6_k}
