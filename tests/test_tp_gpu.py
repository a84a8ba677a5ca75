"""Tensor-parallel decode with the gather fused into the product kernel, through the C ABI.

On one GPU the ranks of a group are stood in for by launches that run one after another on one stream with every
"peer" buffer on the same device, so no kernel ever waits for another kernel. With two or more GPUs the same calls
run as one process per GPU over inter-process mappings."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from test_decode_gpu import bf16_dev, make_linear

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def sharded_reference(gpu, w, x, ranks, splits, tokens, round_z):
    """Per-rank qtip_multiply into a local buffer, z concatenated by hand, output transform on the full width."""
    lin = gpu.linear
    n_in, n_out = w.n_in, w.n_out
    rows = n_out // ranks
    rot = torch.empty((tokens, n_in), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(tokens * max(n_in, n_out), dtype=torch.float32, device="cuda")
    lin.qtip_prepare(w, x, scratch, rot, tokens)
    z = torch.zeros((splits, tokens, n_out), dtype=torch.float32, device="cuda")
    for r in range(ranks):
        zl = torch.zeros((splits, tokens, rows), dtype=torch.float32, device="cuda")
        lin.qtip_multiply_batch(w.rows(r * rows, rows), rot, zl, rows, splits, tokens, 0)  # the kernel the push uses
        z[:, :, r * rows:(r + 1) * rows] = zl
    y = torch.empty((tokens, n_out), dtype=torch.bfloat16, device="cuda")
    lin.qtip_finish(w, z, y, scratch, round_z, splits, tokens)
    return y


@pytest.mark.parametrize("ranks,tokens,splits", [(2, 1, 1), (4, 1, 2), (8, 1, 1), (2, 5, 1), (4, 24, 2), (8, 16, 1)])
def test_push_and_gather_match_the_sharded_products(gpu, ranks, tokens, splits):
    n_in, n_out = 1536, 2048
    w, *_ = make_linear(gpu, n_in, n_out, 300 + ranks, sv_scale=0.02)
    rows = n_out // ranks
    group = gpu.tp.Exchange.local_group(ranks, n_out, max_tokens=tokens, max_splits=splits)
    try:
        rot = torch.empty((tokens, n_in), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(tokens * max(n_in, n_out), dtype=torch.float32, device="cuda")
        for step in range(5):  # both slots, several epochs
            xb = gpu.synth.f32_to_bf16_bits(
                (np.random.default_rng(step).standard_normal((tokens, n_in)) * 0.3).astype(np.float32))
            x = bf16_dev(xb)
            round_z = step % 2 == 1
            want = sharded_reference(gpu, w, x, ranks, splits, tokens, round_z)
            slot = step & 1
            gpu.linear.qtip_prepare(w, x, scratch, rot, tokens)
            for r in range(ranks):  # every rank's push completes before any wait is launched (one stream)
                group[r].multiply_push(w.rows(r * rows, rows), rot, slot, n_out, r * rows, splits, tokens)
            for r in range(ranks):
                z = group[r].gather_wait(slot)
                y = torch.empty((tokens, n_out), dtype=torch.bfloat16, device="cuda")
                gpu.linear.qtip_finish(w, z, y, scratch, round_z, splits, tokens)
                assert torch.equal(y.view(torch.int16), want.view(torch.int16)), (step, r)
                group[r].check()
    finally:
        for r, ex in enumerate(group):
            ex.close(free_local=True)


def test_wait_for_a_push_that_never_comes_runs_out(gpu):
    """Rank 1 never pushes: rank 0's wait gives up after about a second, reports it, and the context stays usable."""
    n_in, n_out = 512, 256
    w, *_ = make_linear(gpu, n_in, n_out, 17)
    group = gpu.tp.Exchange.local_group(2, n_out)
    try:
        rot = torch.zeros(n_in, dtype=torch.bfloat16, device="cuda")
        group[0].multiply_push(w.rows(0, 128), rot, 0, n_out, 0)
        group[0].gather_wait(0)
        with pytest.raises(gpu.QtipError):
            group[0].check()
        torch.cuda.synchronize()
        assert float(torch.ones(4, device="cuda").sum()) == 4.0
    finally:
        for ex in group:
            ex.close()


def test_exchange_argument_checks(gpu):
    n_in, n_out = 512, 256
    w, *_ = make_linear(gpu, n_in, n_out, 18)
    group = gpu.tp.Exchange.local_group(2, n_out)
    try:
        rot = torch.zeros(n_in, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(gpu.QtipError):
            group[0].multiply_push(w.rows(0, 128), rot, 2, n_out, 0)  # slot
        with pytest.raises(gpu.QtipError):
            group[0].multiply_push(w.rows(0, 128), rot, 0, n_out, 192)  # rows beyond the matrix
        with pytest.raises(gpu.QtipError):
            group[0].multiply_push(w.rows(0, 128), rot, 0, n_out, 0, 1, 4)  # more tokens than the exchange holds
    finally:
        for ex in group:
            ex.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_over_peer_memory():
    """One process per GPU, gloo for the set-up exchange; every rank checks its y against the unsharded operator."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29611")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29611", os.path.join(ROOT, "tests", "tp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert out.stdout.count("tp worker ok") == 2
