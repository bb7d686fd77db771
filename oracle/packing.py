"""numpy block packers and seeded synthetic-weight generators (test infrastructure).

Block layouts follow the reference, not upstream ggml where the two differ:
  Q8_0  {f16 d; i8 qs[32]}                      crates/kernels/shaders/gemv_q8_0.metal:11-14
  Q4_0  {f16 d; u8 qs[16]}, low nibble = element 2i, high nibble = element 2i+1
                                                crates/kernels/shaders/gemv_q4_0.metal:10-15
  Q4_K  {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]}; pair j: elements 64j..64j+31 are the low
        nibbles of qs[32j..] with scale/min index j, elements 64j+32..64j+63 the high nibbles
        with index j+4            crates/kernels/shaders/dequant.metal:74-82, gemv_q4k.metal:47-80
The value distributions are the ones the benchmark configurations state.
"""
from __future__ import annotations

import numpy as np

__all__ = ["pack_q8_0", "pack_q4_0", "pack_q4k", "pack_q4k_scales", "rand_q8_0", "rand_q4_0",
           "rand_q4k", "rand_weights", "lcg_random_f32", "pack_q5_0", "pack_q5k", "pack_q6k", "rand_q5_0", "rand_q5k", "rand_q6k"]


def pack_q8_0(d: np.ndarray, qs: np.ndarray) -> np.ndarray:
    """d: [m, nb] (rounded to f16); qs: [m, nb, 32] int8 -> uint8 [m, nb*34]."""
    m, nb = d.shape
    out = np.empty((m, nb, 34), np.uint8)
    out[:, :, 0:2] = d.astype(np.float16).view(np.uint8).reshape(m, nb, 2)
    out[:, :, 2:] = qs.astype(np.int8).view(np.uint8).reshape(m, nb, 32)
    return out.reshape(m, nb * 34)


def pack_q4_0(d: np.ndarray, nib: np.ndarray) -> np.ndarray:
    """d: [m, nb]; nib: [m, nb, 32] in 0..15 (value = nib - 8) -> uint8 [m, nb*18]."""
    m, nb = d.shape
    nib = nib.astype(np.uint8).reshape(m, nb, 16, 2)
    out = np.empty((m, nb, 18), np.uint8)
    out[:, :, 0:2] = d.astype(np.float16).view(np.uint8).reshape(m, nb, 2)
    out[:, :, 2:] = nib[..., 0] | (nib[..., 1] << 4)
    return out.reshape(m, nb * 18)


def pack_q4k_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Inverse of get_scale_min_k4 (crates/engine/src/forward.rs:359-369): [.., 8] x2 -> [.., 12]."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    s = np.empty(sc.shape[:-1] + (12,), np.uint8)
    s[..., 0:4] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    s[..., 4:8] = mn[..., 0:4] | ((mn[..., 4:8] >> 4) << 6)
    s[..., 8:12] = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    return s


def pack_q4k(d, dmin, sc, mn, nib) -> np.ndarray:
    """d, dmin: [m, nb]; sc, mn: [m, nb, 8] in 0..63; nib: [m, nb, 256] in 0..15 -> [m, nb*144]."""
    m, nb = d.shape
    out = np.empty((m, nb, 144), np.uint8)
    out[:, :, 0:2] = d.astype(np.float16).view(np.uint8).reshape(m, nb, 2)
    out[:, :, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(m, nb, 2)
    out[:, :, 4:16] = pack_q4k_scales(sc, mn)
    n = nib.astype(np.uint8).reshape(m, nb, 4, 2, 32)  # [pair j][low/high half][l]
    out[:, :, 16:] = (n[:, :, :, 0, :] | (n[:, :, :, 1, :] << 4)).reshape(m, nb, 128)
    return out.reshape(m, nb * 144)


def rand_q8_0(rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    """int8 uniform in [-127, 127]; d = f16(|N(0, 0.02)| / 127)."""
    nb = k // 32
    d = np.abs(rng.normal(0.0, 0.02, (m, nb))) / 127.0
    qs = rng.integers(-127, 128, (m, nb, 32), dtype=np.int8)
    return pack_q8_0(d, qs)


def rand_q4_0(rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    """nibbles uniform in 0..15; d = f16(|N(0, 0.02)| / 8) (the scale law is this build's choice)."""
    nb = k // 32
    d = np.abs(rng.normal(0.0, 0.02, (m, nb))) / 8.0
    nib = rng.integers(0, 16, (m, nb, 32), dtype=np.uint8)
    return pack_q4_0(d, nib)


def rand_q4k(rng: np.random.Generator, m: int, k: int, sigma: float = 0.01) -> np.ndarray:
    """d, dmin = f16(|N(0, sigma)|); 6-bit scale/min uniform in 0..63; nibbles uniform in 0..15."""
    nb = k // 256
    d = np.abs(rng.normal(0.0, sigma, (m, nb)))
    dmin = np.abs(rng.normal(0.0, sigma, (m, nb)))
    sc = rng.integers(0, 64, (m, nb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, (m, nb, 8), dtype=np.uint8)
    nib = rng.integers(0, 16, (m, nb, 256), dtype=np.uint8)
    return pack_q4k(d, dmin, sc, mn, nib)


def pack_q5_0(d: np.ndarray, q: np.ndarray) -> np.ndarray:
    """d: [m, nb]; q: [m, nb, 32] in 0..31 (value = d * (q - 16)) -> uint8 [m, nb*22].
    Layout the reference decodes (crates/engine/src/forward.rs:900-919): byte j of qs = element j (low nibble) and
    element j + 16 (high nibble); fifth bit of element e = bit e of the 32-bit little-endian word qh."""
    m, nb = d.shape
    q = q.astype(np.uint32).reshape(m, nb, 32)
    out = np.empty((m, nb, 22), np.uint8)
    out[:, :, 0:2] = d.astype(np.float16).view(np.uint8).reshape(m, nb, 2)
    qh = ((q >> 4) << np.arange(32, dtype=np.uint32)).sum(-1).astype(np.uint32)
    out[:, :, 2:6] = qh.view(np.uint8).reshape(m, nb, 4)
    out[:, :, 6:] = ((q[:, :, :16] & 15) | ((q[:, :, 16:] & 15) << 4)).astype(np.uint8)
    return out.reshape(m, nb * 22)


def pack_q5k(d, dmin, sc, mn, q) -> np.ndarray:
    """d, dmin: [m, nb]; sc, mn: [m, nb, 8] in 0..63; q: [m, nb, 256] in 0..31 -> [m, nb*176].
    Q4_K's layout with 32 bytes of fifth bits after the scales: bit e % 8 of qh[e / 8] belongs to element e
    (crates/engine/src/forward.rs:979-1012)."""
    m, nb = d.shape
    q = q.astype(np.uint8).reshape(m, nb, 256)
    out = np.empty((m, nb, 176), np.uint8)
    out[:, :, 0:2] = d.astype(np.float16).view(np.uint8).reshape(m, nb, 2)
    out[:, :, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(m, nb, 2)
    out[:, :, 4:16] = pack_q4k_scales(sc, mn)
    out[:, :, 16:48] = np.packbits((q >> 4).reshape(m, nb, 32, 8), axis=-1, bitorder="little").reshape(m, nb, 32)
    n = (q & 15).reshape(m, nb, 4, 2, 32)
    out[:, :, 48:] = (n[:, :, :, 0, :] | (n[:, :, :, 1, :] << 4)).reshape(m, nb, 128)
    return out.reshape(m, nb * 176)


def pack_q6k(d, sc, q) -> np.ndarray:
    """d: [m, nb]; sc: [m, nb, 16] int8; q: [m, nb, 256] in -32..31 -> [m, nb*210] as the reference decodes it
    (crates/engine/src/forward.rs:920-949): per half h of 128 elements and l < 32, ql[64h + l] holds the low nibbles of
    elements 128h + l (low) and 128h + l + 64 (high), ql[64h + l + 32] those of 128h + l + 32 and 128h + l + 96, and
    qh[32h + l] the two upper bits of the four, lowest pair first."""
    m, nb = d.shape
    u = (q.astype(np.int32) + 32).astype(np.uint8).reshape(m, nb, 2, 4, 32)      # [half][group of 32][l]
    out = np.empty((m, nb, 210), np.uint8)
    ql = np.empty((m, nb, 2, 2, 32), np.uint8)
    ql[:, :, :, 0, :] = (u[:, :, :, 0, :] & 15) | ((u[:, :, :, 2, :] & 15) << 4)
    ql[:, :, :, 1, :] = (u[:, :, :, 1, :] & 15) | ((u[:, :, :, 3, :] & 15) << 4)
    out[:, :, 0:128] = ql.reshape(m, nb, 128)
    qh = (u[:, :, :, 0, :] >> 4) | ((u[:, :, :, 1, :] >> 4) << 2) | ((u[:, :, :, 2, :] >> 4) << 4) | ((u[:, :, :, 3, :] >> 4) << 6)
    out[:, :, 128:192] = qh.reshape(m, nb, 64)
    out[:, :, 192:208] = sc.astype(np.int8).view(np.uint8).reshape(m, nb, 16)
    out[:, :, 208:210] = d.astype(np.float16).view(np.uint8).reshape(m, nb, 2)
    return out.reshape(m, nb * 210)


def rand_q5_0(rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    """5-bit values uniform in 0..31; d = f16(|N(0, 0.02)| / 16)."""
    nb = k // 32
    return pack_q5_0(np.abs(rng.normal(0.0, 0.02, (m, nb))) / 16.0, rng.integers(0, 32, (m, nb, 32), dtype=np.uint8))


def rand_q5k(rng: np.random.Generator, m: int, k: int, sigma: float = 0.01) -> np.ndarray:
    nb = k // 256
    return pack_q5k(np.abs(rng.normal(0.0, sigma, (m, nb))), np.abs(rng.normal(0.0, sigma, (m, nb))),
                    rng.integers(0, 64, (m, nb, 8), dtype=np.uint8), rng.integers(0, 64, (m, nb, 8), dtype=np.uint8),
                    rng.integers(0, 32, (m, nb, 256), dtype=np.uint8))


def rand_q6k(rng: np.random.Generator, m: int, k: int, sigma: float = 0.001) -> np.ndarray:
    """6-bit values uniform in -32..31; int8 sub-block scales uniform in -128..127; d = f16(|N(0, sigma)|)."""
    nb = k // 256
    return pack_q6k(np.abs(rng.normal(0.0, sigma, (m, nb))), rng.integers(-128, 128, (m, nb, 16)).astype(np.int8),
                    rng.integers(-32, 32, (m, nb, 256)).astype(np.int8))


def rand_weights(fmt: int, rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    return (rand_q8_0, rand_q4_0, rand_q4k, rand_q5_0, rand_q5k, rand_q6k)[fmt](rng, m, k)


def lcg_random_f32(n: int, seed: int) -> np.ndarray:
    """The reference tests' input generator (crates/kernels/src/dispatch.rs:1805-1813):
    state = state*6364136223846793005 + 1442695040888963407 (mod 2^64), value =
    f32(state >> 33) / f32(u32::MAX) * 2 - 1."""
    out = np.empty(n, np.float32)
    state = seed & 0xFFFFFFFFFFFFFFFF
    umax = np.float32(4294967295.0)
    for i in range(n):
        state = (state * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(state >> 33) / umax * np.float32(2.0) - np.float32(1.0)
    return out
