"""Seeded synthetic inputs of the benchmark configurations (numpy PCG64), shared by the tests and the benchmark so
that both sides of every comparison read the same arrays."""
import numpy as np


def seeded_tlut(seed=1):
    """[512, 2] fp16 codebook: N(0,1) entries scaled to unit rms, rounded to fp16."""
    t = np.random.default_rng(seed).standard_normal((512, 2))
    t /= np.sqrt(np.mean(t * t))
    return t.astype(np.float16)


def gaussian_matrix(rows, cols, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(scale)).astype(np.float32)


def tile_sequences(W):
    """Rows-by-columns fp32 matrix -> [tiles, 256] sequences: tile (tr, tc) in row-major tile order, weights ordered by
    the codec's tile permutation (sequence position p holds tile element perm[p] = 16 r + c)."""
    m, n = W.shape
    perm = tile_perm()
    t = W.reshape(m // 16, 16, n // 16, 16).transpose(0, 2, 1, 3).reshape(-1, 256)
    return np.ascontiguousarray(t[:, perm])


def tile_perm():
    p = np.arange(256)
    e, a, c, d, b = p & 1, (p >> 1) & 1, (p >> 2) & 1, (p >> 3) & 3, (p >> 5) & 7
    return a * 128 + b * 16 + c * 8 + d * 2 + e


def random_trellis(n_out, n_in, seed):
    """Uniform uint16 code words, interpreted directly as the kernel layout."""
    rng = np.random.default_rng(seed)
    return rng.integers(0, 65536, size=(n_out // 16) * (n_in // 16) * 32, dtype=np.uint16)


def signs(n, seed):
    return (np.random.default_rng(seed).integers(0, 2, size=n) * 2 - 1).astype(np.float32)


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def spd_hessian(n, seed, rank=64):
    """Small-scale stand-in of the activation Hessian: H = X^T X / N for X = Z + Zr C with a rank-`rank` correlated
    part, plus 1e-2 * mean(diag) damping. fp64."""
    rng = np.random.default_rng(seed)
    N = 4 * n
    X = rng.standard_normal((N, n)) + rng.standard_normal((N, rank)) @ (rng.standard_normal((rank, n)) / 8.0)
    H = X.T @ X / N
    H += 1e-2 * np.mean(np.diag(H)) * np.eye(n)
    return H


def reference_signs(seed, count):
    """+-1 signs of the reference's deterministic generator (`Rng::sign`, src/common.hpp:91-107: splitmix64 seeded with
    seed * 0x9E3779B97F4A7C15 + 0x1234567, sign = top bit of each output), so that SU / SV made here equal the
    reference quantizer's for the same seed (SU: seed; SV of linear i: seed * 1000003 + i + 1,
    src/quantizer.cpp:128-130,208-212)."""
    M = (1 << 64) - 1
    s = (seed * 0x9E3779B97F4A7C15 + 0x1234567) & M
    out = np.empty(count, np.float32)
    for i in range(count):
        s = (s + 0x9E3779B97F4A7C15) & M
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        z ^= z >> 31
        out[i] = -1.0 if (z >> 63) else 1.0
    return out
