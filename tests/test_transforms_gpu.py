"""Hadamard transforms, elementwise kernels and the LDLQ feedback kernels against the oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import golden
from test_viterbi_gpu import dev, u16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [96, 160, 1024, 12288, 28672])
def test_hadamard_rows_vs_reference_vectors(gpu, n):
    """fp32 in-place row transform vs the reference's fp64 vectors; tolerance 2e-5 absolute as the reference's own GPU
    test (values are O(1))."""
    g = golden("hadamard_ref.npz")
    x = g["x_%d" % n]
    for t, key in ((0, "u"), (1, "ut")):
        X = dev(x.astype(np.float32))
        gpu.codec.k_hadamard_rows(X, x.shape[0], n, n, t)
        assert np.abs(X.cpu().numpy() - g["%s_%d" % (key, n)]).max() < 2e-5


def test_hadamard_rows_strided_and_large(gpu, oracle):
    rng = np.random.default_rng(3)
    rows, n, ld = 5, 384, 400
    buf = rng.standard_normal((rows, ld)).astype(np.float32)
    X = dev(buf)
    gpu.codec.k_hadamard_rows(X, rows, n, ld, 1)
    out = X.cpu().numpy()
    ref = oracle.hadamard_rows(buf[:, :n].astype(np.float64), True)
    assert np.abs(out[:, :n] - ref).max() < 2e-5
    assert np.array_equal(out[:, n:], buf[:, n:])  # padding untouched
    x = rng.standard_normal((2, 57344)).astype(np.float32)  # the longest supported row (28 x 2048)
    X = dev(x)
    gpu.codec.k_hadamard_rows(X, 2, 57344, 57344, 0)
    assert np.abs(X.cpu().numpy() - oracle.hadamard_rows(x.astype(np.float64), False)).max() < 2e-5
    with pytest.raises(gpu.QtipError) as e:
        gpu.codec.k_hadamard_rows(dev(np.zeros((1, 100), np.float32)), 1, 100, 100, 0)
    assert e.value.code == -2


def test_elementwise_kernels(gpu):
    rng = np.random.default_rng(4)
    rows, cols, ld = 37, 53, 64
    A = rng.standard_normal((rows, ld)).astype(np.float32)
    B = rng.standard_normal((rows, ld)).astype(np.float32)
    rs, cs = rng.standard_normal(rows).astype(np.float32), rng.standard_normal(cols).astype(np.float32)
    c = gpu.codec
    X = dev(A)
    c.k_scale_rows_cols(X, rows, cols, ld, dev(rs), dev(cs))
    assert np.array_equal(X.cpu().numpy()[:, :cols], (A[:, :cols] * rs[:, None]) * cs[None, :])
    X = dev(A)
    c.k_scale(X, rows, cols, ld, 0.37)
    assert np.array_equal(X.cpu().numpy()[:, :cols], A[:, :cols] * np.float32(0.37))
    D = torch.zeros_like(X)
    c.k_sub(dev(A), dev(B), D, rows, cols, ld)
    assert np.array_equal(D.cpu().numpy()[:, :cols], A[:, :cols] - B[:, :cols])
    T = torch.zeros((cols, rows), dtype=torch.float32, device="cuda")
    c.k_transpose(dev(A), rows, cols, ld, T, rows)
    assert np.array_equal(T.cpu().numpy(), A[:, :cols].T)
    acc = torch.zeros(1, dtype=torch.float64, device="cuda")
    c.k_sumsq(dev(A), rows, cols, ld, acc)
    assert abs(float(acc) - float((A[:, :cols].astype(np.float64) ** 2).sum())) < 1e-9
    acc.zero_()
    c.k_dot(dev(A), ld, dev(B), ld, rows, cols, acc)
    assert abs(float(acc) - float((A[:, :cols].astype(np.float64) * B[:, :cols]).sum())) < 1e-9
    H = rng.standard_normal((40, 40)).astype(np.float32)
    Hd = dev(H)
    c.k_add_diag(Hd, 40, 0.5)
    assert np.array_equal(np.diag(Hd.cpu().numpy()), np.diag(H) + np.float32(0.5))
    acc.zero_()
    c.k_diag_sum(dev(H), 40, acc)
    assert abs(float(acc) - float(np.diag(H).astype(np.float64).sum())) < 1e-12
    hi = torch.zeros((rows, cols), dtype=torch.int16, device="cuda")
    lo = torch.zeros((rows, cols), dtype=torch.int16, device="cuda")
    c.k_diff_split_bf16(dev(A), dev(B), rows, cols, ld, hi, lo, cols)
    v = A[:, :cols] - B[:, :cols]
    h = gpu.synth.f32_to_bf16_bits(v)
    assert np.array_equal(u16(hi), h)
    assert np.array_equal(u16(lo), gpu.synth.f32_to_bf16_bits(v - gpu.synth.bf16_bits_to_f32(h)))
    c.k_split_bf16(dev(A), rows, cols, ld, hi, None, cols)
    assert np.array_equal(u16(hi), gpu.synth.f32_to_bf16_bits(A[:, :cols]))


def test_pack_and_kernel_layout_vs_reference_vectors(gpu):
    g = golden("pack_ref.npz")
    m, n = int(g["m"]), int(g["n"])
    c = gpu.codec
    pk = c.pack_trellis(dev(g["states"]))
    assert np.array_equal(u16(pk), g["packed"])
    sw = c.swizzle_for_kernel(pk, m, n)
    assert np.array_equal(u16(sw), g["kernel"])
    assert np.array_equal(u16(c.unpack_trellis(c.unswizzle_for_kernel(sw, m, n))), g["states"])
    with pytest.raises(gpu.QtipError):
        c.swizzle_for_kernel(pk, 48, 96)


def ldlq_problem(oracle, m, n, seed):
    rng = np.random.default_rng(seed)
    Wr = rng.standard_normal((m, n)).astype(np.float32)
    G = rng.standard_normal((n, 2 * n)) * (1.0 + (np.arange(2 * n) % 7))[None, :] ** 0.5
    H = G @ G.T / (2 * n) + 0.05 * np.eye(n)
    return Wr, H, oracle.block_ldl(H)


def test_ldlq_prep_bit_exact(gpu, oracle):
    rng = np.random.default_rng(8)
    n, m = 256, 48
    WT = rng.standard_normal((n, m)).astype(np.float32)
    hatWT = (WT + 0.1 * rng.standard_normal((n, m))).astype(np.float32)
    prod = (0.05 * rng.standard_normal((n, m))).astype(np.float32)
    L = np.tril(rng.standard_normal((n, n)) * 0.1, -16).astype(np.float32)
    for col0, bufend in ((240, 256), (128, 256), (176, 256), (0, 128)):
        X = torch.zeros((m // 16, 256), dtype=torch.float32, device="cuda")
        gpu.codec.k_ldlq_prep(dev(WT), dev(hatWT), dev(prod), dev(L), n, m, col0, bufend, X)
        assert np.array_equal(X.cpu().numpy(), oracle.ldlq_prep(WT, hatWT, prod, L, col0, bufend))
    with pytest.raises(gpu.QtipError):
        gpu.codec.k_ldlq_prep(dev(WT), dev(hatWT), dev(prod), dev(L), n, m, 0, 256, X)


def test_ldlq_bit_exact_vs_restated_schedule(gpu, oracle, hyb):
    """m = 64, n = 256 (the reference's LDLQ test size): states and hatW bit-identical to the fp32 restatement of the
    device schedule; proxy error within 1 % of the fp64 port of the upstream algorithm; decode(states) == hatW."""
    tl, lut, _ = hyb
    m, n = 64, 256
    Wr, H, L = ldlq_problem(oracle, m, n, 21)
    WT = np.ascontiguousarray(Wr.T)
    lut_d, _ = gpu.codec.device_lut(tl)
    hat_d = torch.empty((n, m), dtype=torch.float32, device="cuda")
    Q_d = torch.zeros(((m // 16) * (n // 16), 128), dtype=torch.int16, device="cuda")
    ws = gpu.codec.ldlq_gpu(dev(WT), dev(L), n, m, hat_d, Q_d, lut_d)
    torch.cuda.synchronize()
    ohat, oQ = oracle.ldlq_f32(WT, L, lut)
    assert np.array_equal(u16(Q_d), oQ)
    assert np.array_equal(hat_d.cpu().numpy(), ohat)
    hat64, Q64 = oracle.ldlq_ref(Wr, L, lut)

    def proxy(hat):
        D = (Wr - hat).astype(np.float64)
        return np.trace(D @ H @ D.T) / np.trace(Wr.astype(np.float64) @ H @ Wr.T.astype(np.float64))

    pg, pr = proxy(hat_d.cpu().numpy().T), proxy(hat64)
    assert abs(pg - pr) / pr < 0.01
    # row-block sharding: quantising rows [16, 48) alone gives the same codes for those rows
    hat2 = torch.full((n, m), 7.0, dtype=torch.float32, device="cuda")
    Q2 = torch.zeros_like(Q_d)
    gpu.codec.ldlq_gpu(dev(WT), dev(L), n, m, hat2, Q2, lut_d, workspace=ws, j0=16, mj=32)
    torch.cuda.synchronize()
    nb = n // 16
    assert np.array_equal(u16(Q2)[nb:3 * nb], oQ[nb:3 * nb])
    assert np.array_equal(hat2.cpu().numpy()[:, 16:48], ohat[:, 16:48])
    assert bool((hat2[:, :16] == 7.0).all()) and bool((hat2[:, 48:] == 7.0).all())


def test_quantize_linear_round_trip_through_the_runtime_operator(gpu, oracle):
    """Encode side meets decode side: a 64 x 384 linear is rotated, LDLQ-quantised, packed into the checkpoint layout,
    and the runtime operator on those tensors must reproduce y = W_hat x, where W_hat is the encoder's own
    reconstruction diag(SV) T_m (hatWr Wscale) T_n^T diag(SU). Also: LDLQ beats plain nearest-path quantisation in the
    Hessian-weighted proxy error, and the device rotation agrees with the fp64 transform."""
    s = gpu.synth
    m, n = 64, 384
    rng = np.random.default_rng(33)
    W = (0.02 * rng.standard_normal((m, n))).astype(np.float32)
    H = s.spd_hessian(n, 34)
    su, sv = s.signs(n, 7), s.signs(m, 8)
    tl = s.seeded_tlut(1)
    lut_d, lut_rms = gpu.codec.device_lut(tl)
    HRr, creg = gpu.codec.rotate_hessian(dev(H.astype(np.float32)), dev(su))
    Href = oracle.hadamard_rows(oracle.hadamard_rows((H + creg * np.eye(n)) * su[None, :] * su[:, None], True).T.copy(), True)
    assert np.abs(HRr.cpu().numpy() - Href).max() < 2e-5 * max(1.0, np.abs(Href).max())
    Hs = 0.5 * (Href + Href.T)
    L = oracle.block_ldl(Hs)
    out = gpu.codec.quantize_linear(dev(W), dev(L), dev(su), dev(sv), lut_d, lut_rms)
    torch.cuda.synchronize()
    WT, hatWT = out["WT"], out["hatWT"]
    Wr_ref = oracle.hadamard_rows(oracle.hadamard_rows((W * sv[:, None] * su[None, :]).astype(np.float64), True).T.copy(), True)
    assert np.abs(WT.cpu().numpy() * out["wscale"] - Wr_ref).max() < 2e-5
    # proxy error: LDLQ (with feedback) vs the same quantiser without feedback (identity Hessian)
    p_ldlq = gpu.codec.proxy_error(WT, hatWT, dev(Hs.astype(np.float32)))
    hat0 = torch.empty_like(WT)
    Q0 = torch.empty_like(out["Q"])
    gpu.codec.ldlq_gpu(WT, torch.zeros((n, n), dtype=torch.float32, device="cuda"), n, m, hat0, Q0, lut_d)
    p_plain = gpu.codec.proxy_error(WT, hat0, dev(Hs.astype(np.float32)))
    assert p_ldlq < p_plain and p_ldlq < 0.2
    # decode the checkpoint tensors with the oracle and compare with the encoder's hatWT (fp16 LUT values, exact)
    tr = out["trellis"].cpu().numpy().view(np.uint16).reshape(-1)
    dec = oracle.decode_rows(tr, n, m, tl.view(np.uint16), 0, m, False)
    assert np.array_equal(dec, hatWT.cpu().numpy().T)
    # runtime operator on the written tensors vs the dense reconstruction
    w = gpu.linear.Matrix(out["trellis"].view(-1), dev(su), out["SV"].contiguous(), gpu.linear.runtime_lut(tl), n, m)
    x = (rng.standard_normal(n) * 0.1).astype(np.float32)
    xb = s.f32_to_bf16_bits(x)
    y = torch.empty(m, dtype=torch.bfloat16, device="cuda")
    rot = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    z = torch.empty(m, dtype=torch.float32, device="cuda")
    gpu.linear.qtip_forward(w, torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16), y,
                            torch.empty(n, dtype=torch.float32, device="cuda"), rot, z, False, 1)
    What = sv[:, None] * oracle.hadamard_rows(oracle.hadamard_rows(dec.astype(np.float64) * out["wscale"], False).T.copy(),
                                              False).T * su[None, :]
    y_ref = What @ s.bf16_bits_to_f32(xb).astype(np.float64)
    err = np.linalg.norm(y.float().cpu().numpy() - y_ref) / np.linalg.norm(y_ref)
    assert err < 2e-2, err  # bf16 LUT, bf16 rotated input and bf16 output against an fp64 dense product
    assert np.linalg.norm(What - W) / np.linalg.norm(W) < 0.5  # 2 bits per weight: the reconstruction is W-like


def test_quantize_linear_as_one_call_matches_the_assembled_steps(gpu, oracle):
    """qtip_quantize_linear against the same steps issued one by one from the host mirror: every output bit for bit."""
    s = gpu.synth
    m, n = 96, 256
    rng = np.random.default_rng(55)
    W = (0.03 * rng.standard_normal((m, n))).astype(np.float32)
    H = s.spd_hessian(n, 56)
    su, sv = s.signs(n, 9), s.signs(m, 10)
    lut_d, lut_rms = gpu.codec.device_lut(s.seeded_tlut(1))
    HRr, _ = gpu.codec.rotate_hessian(dev(H.astype(np.float32)), dev(su))
    Hs = HRr.cpu().numpy().astype(np.float64)
    L = dev(oracle.block_ldl(0.5 * (Hs + Hs.T)))
    a = gpu.codec.quantize_linear(dev(W), L, dev(su), dev(sv), lut_d, lut_rms)
    b = gpu.codec.quantize_linear_fused(dev(W), L, dev(su), dev(sv), lut_d, lut_rms)
    b["workspace"].check()
    assert a["wscale"] == b["wscale"]
    for key in ("WT", "hatWT", "Q", "trellis", "SV"):
        assert torch.equal(a[key], b[key]), key
    with pytest.raises(gpu.QtipError):
        gpu.codec.quantize_linear_fused(dev(W[:80]), L, dev(su), dev(sv[:80]), lut_d, lut_rms)  # m % 32 != 0


@pytest.mark.parametrize("slices", [2, 3, 4])
def test_ldlq_row_slices_on_side_streams_give_the_same_codes(gpu, oracle, hyb, slices, monkeypatch):
    """The rows of one call run as 2..4 independent chains on side streams (QTIP_LDLQ_SLICES forces it for this small
    matrix): states and hatW stay bit-identical to the fp32 restatement of the schedule, and the status word is clean."""
    tl, lut, _ = hyb
    m, n = 112, 256  # 7 tile rows: uneven slices
    Wr, H, L = ldlq_problem(oracle, m, n, 23)
    WT = np.ascontiguousarray(Wr.T)
    lut_d, _ = gpu.codec.device_lut(tl)
    monkeypatch.setenv("QTIP_LDLQ_SLICES", str(slices))
    hat_d = torch.empty((n, m), dtype=torch.float32, device="cuda")
    Q_d = torch.zeros(((m // 16) * (n // 16), 128), dtype=torch.int16, device="cuda")
    ws = gpu.codec.ldlq_gpu(dev(WT), dev(L), n, m, hat_d, Q_d, lut_d)
    ws.check()
    ohat, oQ = oracle.ldlq_f32(WT, L, lut)
    assert np.array_equal(u16(Q_d), oQ)
    assert np.array_equal(hat_d.cpu().numpy(), ohat)


def test_rotate_hessian_as_one_call(gpu):
    s = gpu.synth
    n = 384
    H = s.spd_hessian(n, 77).astype(np.float32)
    su = s.signs(n, 3)
    a, ca = gpu.codec.rotate_hessian(dev(H), dev(su))
    b, cb = gpu.codec.rotate_hessian_fused(dev(H), dev(su))
    assert ca == cb and torch.equal(a, b)
