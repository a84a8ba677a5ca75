"""Generates the golden fixtures of this directory by running the REFERENCE's own CPU code (compiled in place by
`make -C oracle ref` from the reference tree) on seeded inputs. Run from the repository root in a container that has
the reference tree; the outputs are committed, the reference is not needed to use them.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.oracle import Reference  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def main():
    R = Reference()
    assert R.available, "build the reference first: make -C oracle ref"
    rng = np.random.default_rng(20251)
    tlut, lut_h2, lut_rms = R.codebook()

    # --- encode: fp64 tail-biting Viterbi of the reference on fp16-representable inputs at three scales
    B = 36
    scale = np.array([0.6, 1.0, 1.6])[np.arange(B) % 3][:, None]
    X = (rng.standard_normal((B, 256)) * scale).astype(np.float16).astype(np.float32)
    X[33] = 0.0                      # all-zero sequence
    X[34] = np.float32(3.5)          # constant, far outside the codebook
    X[35, ::2] = -X[35, ::2]
    st, hat, cost = R.quantize_seqs(X)
    perm, inv = R.perm()
    np.savez(os.path.join(OUT, "viterbi_ref.npz"), tlut_bits=tlut, lut_rms=lut_rms, X=X, states=st, hat=hat,
             cost=cost, perm=perm.astype(np.int16))

    # --- packing and kernel layout (m = 64, n = 96)
    m, n = 64, 96
    T = (m // 16) * (n // 16)
    Xp = rng.standard_normal((T, 256)).astype(np.float16).astype(np.float32)
    stp, _, _ = R.quantize_seqs(Xp)
    packed = R.pack(stp)
    np.savez(os.path.join(OUT, "pack_ref.npz"), m=m, n=n, states=stp, packed=packed, kernel=R.swizzle(packed, m, n),
             unpacked=R.unpack(packed))

    # --- Hadamard transforms (fp64 reference), hadU and hadUt
    had = {}
    for nn, rows in ((96, 2), (1024, 2), (160, 2), (12288, 1), (28672, 1)):
        x = rng.standard_normal((rows, nn))
        had["x_%d" % nn] = x
        had["u_%d" % nn] = R.hadamard_rows(x, False)
        had["ut_%d" % nn] = R.hadamard_rows(x, True)
    for K in (12, 20, 28):
        had["table_%d" % K] = R.had_table(K)
    np.savez(os.path.join(OUT, "hadamard_ref.npz"), **had)

    # --- block LDL
    G = rng.standard_normal((96, 192))
    H = G @ G.T / 192 + 0.05 * np.eye(96)
    np.savez(os.path.join(OUT, "ldl_ref.npz"), H=H, L=R.block_ldl(H))

    # --- decode side: codebook, dense decode and the fp64 reference linear (in = 384 = 12 * 32, out = 256)
    n_in, n_out = 384, 256
    tr = rng.integers(0, 65536, (n_out // 16) * (n_in // 16) * 32, dtype=np.uint16)
    su = rng.choice([-1.0, 1.0], n_in).astype(np.float32)
    sv = (rng.choice([-1.0, 1.0], n_out) * 0.003).astype(np.float32)
    x = (rng.standard_normal((3, n_in)) * 0.1).astype(np.float32)
    c0, c1, b2 = R.runtime_codebook(tlut)
    dec = dict(n_in=n_in, n_out=n_out, trellis=tr, su=su, sv=sv, x=x, c0=c0, c1=c1, bf16x2=b2,
               rows_f16=R.decode_rows(tr, n_in, n_out, tlut, 32, 64, False),
               rows_bf16=R.decode_rows(tr, n_in, n_out, tlut, 32, 64, True))
    for dr in (0, 1):
        for rz in (0, 1):
            dec["y_%d%d" % (dr, rz)] = R.reference_forward(tr, su, sv, tlut, n_in, n_out, x, dr, rz)
    np.savez(os.path.join(OUT, "decode_ref.npz"), **dec)
    for f in sorted(os.listdir(OUT)):
        print("%8d  %s" % (os.path.getsize(os.path.join(OUT, f)), f))


if __name__ == "__main__":
    main()
