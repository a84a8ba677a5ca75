"""Pins the CPU oracle: against the committed golden vectors (made by the reference's own CPU code, see
tests/golden/make_golden.py), against the reference's committed test vectors when the reference tree is present, and
against the reference code itself when it has been compiled in place."""
import os

import numpy as np
import pytest

from conftest import REFVEC, golden


def test_codebook_and_perm(oracle, hyb):
    tl, lut, rms = hyb
    g = golden("viterbi_ref.npz")
    assert abs(rms - float(g["lut_rms"])) < 1e-15
    p, pi = oracle.perm()
    assert np.array_equal(p, g["perm"].astype(np.int32))
    assert np.array_equal(pi[p], np.arange(256))
    # every state with the same sign-folded entry holds the same word (the 1,024-entry compact table is complete)
    s = np.arange(65536, dtype=np.uint64)
    e = ((s * (s + 1)) >> 6) & 1023
    for k in (0, 17, 511, 512, 1023):
        assert len(set(lut[e == k].tolist())) == 1
    # garbage above bit 15 of a state must not change its entry
    assert oracle.lib.qo_lut_entry(0x12345) == oracle.lib.qo_lut_entry(0x2345)


def test_viterbi_fp64_matches_reference_vectors(oracle, hyb):
    tl, lut, _ = hyb
    g = golden("viterbi_ref.npz")
    st, hat, cost = oracle.quantize_seq_ref(g["X"], lut)
    assert np.array_equal(st, g["states"])
    assert np.array_equal(hat, g["hat"])
    assert np.allclose(cost, g["cost"], rtol=0, atol=1e-12)


def test_exact_viterbi_agrees_with_fp64_on_fp16_inputs(oracle, hyb):
    """The kernel-arithmetic restatement reaches the fp64 optimum on the golden inputs (as the reference reports for
    its GPU kernel: identical paths, cost excess 0) and satisfies the trellis invariants."""
    tl, lut, _ = hyb
    g = golden("viterbi_ref.npz")
    st, hat = oracle.quantize_tiles(g["X"], lut)
    same = (st == g["states"]).all(axis=1)
    for b in range(len(st)):
        c_exact = oracle.path_cost(g["X"][b], st[b], lut)
        assert c_exact <= g["cost"][b] * (1 + 2e-3) + 1e-9
        s = st[b].astype(np.uint32)
        assert (s[127] & 0xFFF) == (s[0] >> 4)
        assert np.array_equal((s[:-1] << 4) & 0xFFFF, s[1:] & 0xFFF0)
    assert same.sum() >= len(st) - 3, "exact kernel arithmetic left the fp64 optimum on %d sequences" % (~same).sum()
    assert np.array_equal(oracle.decode_states(st, lut), hat)


def test_staged_equals_fused(oracle, hyb):
    tl, lut, _ = hyb
    X = golden("viterbi_ref.npz")["X"][:5]
    A, fs = oracle.viterbi_fwd(X, None, 1, lut)
    ov = oracle.viterbi_overlap(A, fs)
    A, fs = oracle.viterbi_fwd(X, ov, 0, lut)
    Q = oracle.viterbi_finish(A, fs, lut)
    st, _ = oracle.quantize_tiles(X, lut)
    assert np.array_equal(Q, st)


def test_packing(oracle):
    g = golden("pack_ref.npz")
    m, n = int(g["m"]), int(g["n"])
    pk = oracle.pack(g["states"])
    assert np.array_equal(pk, g["packed"])
    sw = oracle.swizzle(pk, m, n)
    assert np.array_equal(sw, g["kernel"])
    assert np.array_equal(oracle.unpack(oracle.unswizzle(sw, m, n)), g["states"])
    assert np.array_equal(oracle.unpack(pk), g["unpacked"])
    with pytest.raises(ValueError):
        oracle.swizzle(pk[: 4 * 5], 64, 80)


def test_hadamard(oracle):
    g = golden("hadamard_ref.npz")
    for K in (12, 20, 28):
        H = oracle.had_table(K)
        assert np.array_equal(H, g["table_%d" % K])
        assert np.array_equal(H.astype(int) @ H.astype(int).T, K * np.eye(K, dtype=int))
    for n in (96, 160, 1024, 12288, 28672):
        x = g["x_%d" % n]
        assert np.abs(oracle.hadamard_rows(x, False) - g["u_%d" % n]).max() < 1e-12
        assert np.abs(oracle.hadamard_rows(x, True) - g["ut_%d" % n]).max() < 1e-12
        # orthogonality: hadUt inverts hadU
        assert np.abs(oracle.hadamard_rows(oracle.hadamard_rows(x, False), True) - x).max() < 1e-12
    assert oracle.had_K(12288) == 12 and oracle.had_K(28672) == 28 and oracle.had_K(8192) == 1
    assert oracle.had_K(57344) == 28 and oracle.had_K(100) == 0 and oracle.had_K(36 * 64) == 0


def test_block_ldl(oracle):
    g = golden("ldl_ref.npz")
    L = oracle.block_ldl(g["H"])
    assert np.abs(L - g["L"]).max() < 1e-6
    for b in range(6):
        assert not L[16 * b:16 * b + 16, 16 * b:].any()  # diagonal blocks and everything above are zero


def test_decode_side(oracle, hyb):
    tl, _, _ = hyb
    g = golden("decode_ref.npz")
    n_in, n_out = int(g["n_in"]), int(g["n_out"])
    c0, c1, b2 = oracle.runtime_codebook(tl)
    assert np.array_equal(c0, g["c0"]) and np.array_equal(c1, g["c1"]) and np.array_equal(b2, g["bf16x2"])
    assert np.array_equal(oracle.decode_rows(g["trellis"], n_in, n_out, tl, 32, 64, False), g["rows_f16"])
    assert np.array_equal(oracle.decode_rows(g["trellis"], n_in, n_out, tl, 32, 64, True), g["rows_bf16"])
    for dr in (0, 1):
        for rz in (0, 1):
            y = oracle.reference_forward(g["trellis"], g["su"], g["sv"], tl, n_in, n_out, g["x"], dr, rz)
            assert np.array_equal(y, g["y_%d%d" % (dr, rz)])
    with pytest.raises(ValueError):
        oracle.decode_rows(g["trellis"], n_in, n_out, tl, 8, 16, False)


def test_ldlq_restatement_matches_fp64_port(oracle, hyb):
    """fp32 restatement of the device schedule vs the fp64 port of the upstream algorithm (m = 32, n = 128):
    decode(states) == hatW exactly and the proxy error within 1 % (the reference's own acceptance test)."""
    tl, lut, _ = hyb
    rng = np.random.default_rng(21)
    m, n = 32, 128
    Wr = rng.standard_normal((m, n)).astype(np.float32)
    G = rng.standard_normal((n, 2 * n)) * (1.0 + (np.arange(2 * n) % 7))[None, :] ** 0.5
    H = G @ G.T / (2 * n) + 0.05 * np.eye(n)
    L = oracle.block_ldl(H)
    hat64, Q64 = oracle.ldlq_ref(Wr, L, lut)
    hatT, Q32 = oracle.ldlq_f32(np.ascontiguousarray(Wr.T), L, lut)
    hat32 = np.ascontiguousarray(hatT.T)

    def proxy(hat):
        D = (Wr - hat).astype(np.float64)
        return np.trace(D @ H @ D.T) / np.trace(Wr.astype(np.float64) @ H @ Wr.T.astype(np.float64))

    p64, p32 = proxy(hat64), proxy(hat32)
    assert abs(p32 - p64) / p64 < 0.01
    p, _ = oracle.perm()
    dec = oracle.decode_states(Q32, lut).reshape(m // 16, n // 16, 256)
    tiles = hat32.reshape(m // 16, 16, n // 16, 16).transpose(0, 2, 1, 3).reshape(m // 16, n // 16, 256)
    assert np.array_equal(dec, tiles[:, :, p])


@pytest.mark.skipif(not os.path.isdir(REFVEC), reason="reference tree not present")
def test_against_reference_committed_vectors(oracle):
    """The reference's own test vectors (tests/refvec of the reference tree)."""
    lutf = np.fromfile(os.path.join(REFVEC, "lut.bin"), np.float32).reshape(2, 65536)
    # recover the fp16 tlut from the expanded table: entry idx of state s, sign bit folded out
    s = np.arange(65536, dtype=np.uint64)
    p = s * (s + 1)
    idx, flip = ((p >> 6) & 511).astype(int), ((p >> 15) & 1).astype(bool)
    tl = np.zeros((512, 2), np.float16)
    tl[idx, 0] = np.where(flip, -lutf[0], lutf[0]).astype(np.float16)
    tl[idx, 1] = lutf[1].astype(np.float16)
    lut, _ = oracle.build_lut(tl.view(np.uint16))
    assert np.array_equal((lut & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32), lutf[0])
    assert np.array_equal((lut >> 16).astype(np.uint16).view(np.float16).astype(np.float32), lutf[1])
    assert np.array_equal(oracle.perm()[0], np.fromfile(os.path.join(REFVEC, "perm.bin"), np.int64))
    X = np.fromfile(os.path.join(REFVEC, "vit_x.bin"), np.float32).reshape(-1, 256)
    st_py = np.fromfile(os.path.join(REFVEC, "vit_states.bin"), np.int32).reshape(-1, 128).astype(np.uint16)
    hat_py = np.fromfile(os.path.join(REFVEC, "vit_hat.bin"), np.float32).reshape(-1, 256)
    st, hat = oracle.quantize_tiles(X, lut)  # the exact kernel arithmetic
    assert np.array_equal(st, st_py) and np.array_equal(hat, hat_py)
    st64, hat64, _ = oracle.quantize_seq_ref(X, lut)
    assert np.array_equal(st64, st_py) and np.array_equal(hat64, hat_py)
    ps = np.fromfile(os.path.join(REFVEC, "pack_states.bin"), np.int32).reshape(-1, 128).astype(np.uint16)
    pk = oracle.pack(ps)
    assert np.array_equal(pk.reshape(-1), np.fromfile(os.path.join(REFVEC, "pack_plain.bin"), np.uint16))
    assert np.array_equal(oracle.swizzle(pk, 64, 96).reshape(-1),
                          np.fromfile(os.path.join(REFVEC, "pack_kernel.bin"), np.uint16))
    for n in (96, 1024, 12288, 28672):
        x = np.fromfile(os.path.join(REFVEC, "had_%d_x.bin" % n), np.float64).reshape(4, n)
        for t, nm in ((0, "u"), (1, "ut")):
            ref = np.fromfile(os.path.join(REFVEC, "had_%d_%s.bin" % (n, nm)), np.float64).reshape(4, n)
            assert np.abs(oracle.hadamard_rows(x, t) - ref).max() < 1e-6  # the vectors divide by an fp32 sqrt(n)
    H = np.fromfile(os.path.join(REFVEC, "ldl_H.bin"), np.float64).reshape(96, 96)
    Lr = np.fromfile(os.path.join(REFVEC, "ldl_L.bin"), np.float64).reshape(96, 96)
    assert np.abs(oracle.block_ldl(H) - Lr).max() < 1e-5


def test_against_compiled_reference(oracle, reference, hyb):
    """Oracle vs the reference's C++ on fresh seeded inputs (beyond the committed fixtures)."""
    tl, lut, rms = hyb
    rt, rl, rr = reference.codebook()
    assert np.array_equal(rt, tl) and np.array_equal(rl, lut) and rr == rms
    rng = np.random.default_rng(77)
    X = rng.standard_normal((16, 256)).astype(np.float16).astype(np.float32)
    a = oracle.quantize_seq_ref(X, lut)
    b = reference.quantize_seqs(X)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]) and np.allclose(a[2], b[2], rtol=0, atol=1e-12)
    x = rng.standard_normal((2, 57344))
    assert np.abs(oracle.hadamard_rows(x, True) - reference.hadamard_rows(x, True)).max() < 1e-12
    n_in, n_out = 1024, 128
    tr = rng.integers(0, 65536, (n_out // 16) * (n_in // 16) * 32, dtype=np.uint16)
    su = rng.choice([-1.0, 1.0], n_in).astype(np.float32)
    sv = rng.choice([-1.0, 1.0], n_out).astype(np.float32)
    xx = rng.standard_normal((2, n_in)).astype(np.float32)
    assert np.array_equal(oracle.reference_forward(tr, su, sv, tl, n_in, n_out, xx, True, True),
                          reference.reference_forward(tr, su, sv, tl, n_in, n_out, xx, True, True))
