"""Block LDL of the rotated Hessian on the GPU (qtip_block_ldl) against the CPU oracle's restatement of the reference's
block_ldl_to_L (src/qtip_core.cpp:321-487), against a plain fp64 factorisation, and on a matrix that is not positive
definite."""
import numpy as np
import pytest
import torch

from conftest import golden
from test_viterbi_gpu import dev

pytestmark = pytest.mark.gpu


def block_ldl_f64(A):
    """fp64 yard-stick on the device: Cholesky A = C C^T, L[:, b] = C[:, b] inv(C[b, b]) strictly below block b."""
    n = A.shape[0]
    nb = n // 16
    Cl = torch.linalg.cholesky(A)
    D = torch.stack([Cl[16 * b:16 * b + 16, 16 * b:16 * b + 16] for b in range(nb)])
    cols = Cl.view(n, nb, 16).permute(1, 0, 2).contiguous()
    Lb = torch.linalg.solve_triangular(D, cols, upper=False, left=False)
    L = Lb.permute(1, 0, 2).reshape(n, n).clone()
    rb = torch.arange(n, device=A.device) // 16
    L.masked_fill_(rb[:, None] <= rb[None, :], 0.0)
    return L


def check(gpu, H32, oracle=None, tol64=1e-9):
    Hd = dev(H32)
    L, L64 = gpu.codec.block_ldl(Hd, want_f64=True)
    A = Hd.double()
    A = 0.5 * (A + A.T)
    ref = block_ldl_f64(A)
    err = float((L64 - ref).norm() / max(float(ref.norm()), 1e-300))  # a single block has an all-zero factor
    assert err < tol64, "fp64 factor: relative error %.3g" % err
    assert torch.equal(L, L64.float())
    n = H32.shape[0]
    rb = torch.arange(n, device="cuda") // 16
    assert not bool(L[rb[:, None] <= rb[None, :]].any())  # diagonal blocks and everything above them are zero
    if oracle is not None:
        Lo = oracle.block_ldl(H32.astype(np.float64))
        assert np.abs(L.cpu().numpy() - Lo).max() < 2e-6 * max(1.0, float(np.abs(Lo).max()))
    return L


def test_block_ldl_golden_and_ragged_sizes(gpu, oracle):
    g = golden("ldl_ref.npz")
    H32 = g["H"].astype(np.float32)
    L = check(gpu, H32, oracle)
    assert np.abs(L.cpu().numpy() - g["L"]).max() < 1e-5  # the reference's own vector (made from the fp64 matrix)
    for n, seed in ((16, 3), (144, 4), (272, 5), (1040, 6)):  # one block; sizes that leave partly filled panels and tiles
        check(gpu, gpu.synth.spd_hessian(n, seed).astype(np.float32), oracle)


def test_block_ldl_mid_size_hessian(gpu, oracle):
    """n = 2,048: sixteen panels, trailing updates of up to 15 x 15 tiles; against the oracle and fp64."""
    check(gpu, gpu.synth.spd_hessian(2048, 11).astype(np.float32), oracle)


def test_block_ldl_at_the_q_proj_width(gpu):
    """n = 12,288 (96 panels): a synthetic correlated Hessian made on the device, damped like the quantizer does."""
    n = 12288
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    X = torch.randn(4 * n // 8, n, generator=g, device="cuda") + \
        torch.randn(4 * n // 8, 64, generator=g, device="cuda") @ (torch.randn(64, n, generator=g, device="cuda") / 8.0)
    H = (X.T @ X) / X.shape[0]
    H += 1e-2 * H.diagonal().mean() * torch.eye(n, device="cuda")
    L, L64 = gpu.codec.block_ldl(H, want_f64=True)
    A = H.double()
    A = 0.5 * (A + A.T)
    ref = block_ldl_f64(A)
    assert float((L64 - ref).norm() / ref.norm()) < 1e-8


def test_block_ldl_reports_a_matrix_that_is_not_positive_definite(gpu):
    H = gpu.synth.spd_hessian(256, 2).astype(np.float32)
    H[200, 200] = -1.0
    with pytest.raises(gpu.QtipError) as e:
        gpu.codec.block_ldl(dev(H))
    assert e.value.code == -6
    gpu.codec.block_ldl(dev(gpu.synth.spd_hessian(256, 2).astype(np.float32)))  # the next call starts clean
