"""This repository's LDLQ and group quantizer against the reference's own GPU quantizer (src/quantizer.cpp: ldlq_gpu,
quantize_group; compiled in place for sm_100a), on the same inputs and the same GPU. The two are not bit-comparable:
the reference's cross-buffer update is a split-bf16 library GEMM and its block LDL runs on the host. The acceptance
test is the reference's own (tests/test_gpu.cpp:181-299): proxy error within 1 %, decode(states) == hatW, and the
fraction of identical trellises is reported."""
import numpy as np
import pytest
import torch

from test_viterbi_gpu import dev, u16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refquant(gpu):
    from oracle.oracle import ReferenceQuant
    r = ReferenceQuant()
    if not r.available:
        pytest.skip("the reference's GPU quantizer is not built (make -C oracle refquant)")
    return r


def proxy(W, hat, H):
    D = (W - hat).astype(np.float64)
    Wd = W.astype(np.float64)
    return float(np.einsum("ia,ab,ib->", D, H, D) / np.einsum("ia,ab,ib->", Wd, H, Wd))


@pytest.mark.parametrize("m,n", [(64, 256), (512, 1024)])
def test_ldlq_against_reference_ldlq_gpu(gpu, oracle, refquant, hyb, m, n):
    tl, lut, _ = hyb  # the codebook compiled into the reference
    lut_d, _ = gpu.codec.device_lut(tl)
    rng = np.random.default_rng(21 + m)
    Wr = rng.standard_normal((m, n)).astype(np.float32)
    H = gpu.synth.spd_hessian(n, 5 + m)
    L = oracle.block_ldl(H)
    WT = dev(np.ascontiguousarray(Wr.T))
    Ld = dev(L)
    hat, hat_r = (torch.zeros((n, m), dtype=torch.float32, device="cuda") for _ in range(2))
    Q, Q_r = (torch.zeros(((m // 16) * (n // 16), 128), dtype=torch.int16, device="cuda") for _ in range(2))
    ws = gpu.codec.ldlq_gpu(WT, Ld, n, m, hat, Q, lut_d)
    ws.check()
    refquant.ldlq_gpu(WT.data_ptr(), Ld.data_ptr(), n, m, hat_r.data_ptr(), Q_r.data_ptr())
    torch.cuda.synchronize()
    p_ours = proxy(Wr, hat.cpu().numpy().T, H)
    p_ref = proxy(Wr, hat_r.cpu().numpy().T, H)
    assert abs(p_ours - p_ref) / p_ref < 0.01, "proxy %.6f vs the reference's %.6f" % (p_ours, p_ref)
    same = int((Q == Q_r).all(dim=1).sum())
    print("identical trellises %d / %d, proxy %.6f (reference %.6f)" % (same, Q.shape[0], p_ours, p_ref))
    # the right-most buffer sees no cross-buffer update: its trellises must be identical
    nblk = n // 16
    last = torch.arange(Q.shape[0], device="cuda") % nblk >= nblk - 8
    assert torch.equal(Q[last], Q_r[last])
    # decode(states) == hatW on both sides
    for q, h in ((Q, hat), (Q_r, hat_r)):
        dec = torch.empty((q.shape[0], 256), dtype=torch.float32, device="cuda")
        gpu.codec.k_decode_states(q, q.shape[0], dec, lut_d)
        perm = torch.from_numpy(gpu.synth.tile_perm()).cuda()
        tiles = h.T.reshape(m // 16, 16, nblk, 16).permute(0, 2, 1, 3).reshape(-1, 256)[:, perm]
        assert torch.equal(dec, tiles)


def test_quantize_group_against_reference_quantize_group(gpu, refquant, hyb):
    """Two linears sharing one Hessian, same seed on both sides: identical SU / SV, Wscale to fp32 rounding, proxies
    within 1 %, and the checkpoint words decode to the same hatW the quantizer reports (tests/test_gpu.cpp:301-372)."""
    tl, lut, lut_rms = hyb
    lut_d, rms = gpu.codec.device_lut(tl)
    n, ms, seed = 512, (128, 64), 77
    rng = np.random.default_rng(5)
    Ws = [rng.standard_normal((m, n)).astype(np.float32) * 0.05 for m in ms]
    H = gpu.synth.spd_hessian(n, 9).astype(np.float32)
    ref, timing = refquant.quantize_group(Ws, H, seed)
    su = gpu.synth.reference_signs(seed, n)
    svs = [gpu.synth.reference_signs(seed * 1000003 + i + 1, m) for i, m in enumerate(ms)]
    Hd = dev(H.copy())
    HR, creg = gpu.codec.rotate_hessian_fused(Hd, dev(su))
    L = gpu.codec.block_ldl(HR)
    outs, shared = gpu.codec.quantize_group([dev(w.copy()) for w in Ws], HR, L, dev(su), [dev(s) for s in svs], creg, lut_d,
                                            rms)
    for i, (o, r) in enumerate(zip(outs, ref)):
        assert np.array_equal(u16(o["SU"].view(torch.int16)), r["su_bf16"])
        assert np.array_equal(svs[i], r["sv"])
        assert abs(o["wscale"] - r["wscale"]) <= 2e-6 * r["wscale"]
        assert abs(o["proxy_rot_reg"] - r["proxy_rot_reg"]) / r["proxy_rot_reg"] < 0.01
        assert abs(o["proxy"] - r["proxy"]) / r["proxy"] < 0.01
        same = float(np.mean(np.all(u16(o["trellis"]).reshape(-1, 32) == r["trellis"].reshape(-1, 32), axis=1)))
        print("linear %d: wscale %.6g (ref %.6g), proxy %.5f (ref %.5f), identical trellis words %.3f" %
              (i, o["wscale"], r["wscale"], o["proxy"], r["proxy"], same))
    # the group call equals the one-linear call on the same inputs, bit for bit
    one = gpu.codec.quantize_linear_fused(dev(Ws[0].copy()), L, dev(su), dev(svs[0]), lut_d, rms)
    assert one["wscale"] == outs[0]["wscale"]
    m0 = ms[0]
    assert torch.equal(one["WT"], shared["WT"][:, :m0].contiguous())
