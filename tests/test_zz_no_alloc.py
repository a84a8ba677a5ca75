"""The allocation-free quantisation entry point (for hosts that may not call cudaMalloc: frozen memory pools, plugin
arenas, latency-critical loops). It must give the same bits as qtip_quantize_tiles, on repeated calls that reuse the
library's built-in scratch, and refuse batches larger than that scratch. Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def call_noalloc(gpu, X, lut_d, states, hat):
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    gpu.lib().call("qtip_quantize_tiles_noalloc", C.c_void_p(X.data_ptr()), X.shape[0], C.c_void_p(lut_d.data_ptr()),
                   C.c_void_p(states.data_ptr()), C.c_void_p(hat.data_ptr()), stream)


def test_noalloc_matches_workspace_variant_twice(gpu):
    tl = gpu.synth.seeded_tlut(1)
    lut_d, _ = gpu.codec.device_lut(tl)
    ws = gpu.codec.quantize_workspace(64)
    for seed, B in ((31, 64), (32, 21)):  # second call reuses the scratch the first one dirtied, with a ragged batch
        X = torch.from_numpy(np.random.default_rng(seed).standard_normal((B, 256), dtype=np.float32)).cuda()
        ref_st, ref_hat = gpu.codec.quantize_tiles(X, lut_d, workspace=ws)
        ws.check()
        st = torch.full((B, 128), -1, dtype=torch.int16, device="cuda")
        hat = torch.full((B, 256), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]  # driver-level free memory: sees any cudaMalloc, by anyone
        call_noalloc(gpu, X, lut_d, st, hat)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call allocated device memory"
        assert torch.equal(st, ref_st), "states differ from qtip_quantize_tiles"
        assert torch.equal(hat, ref_hat), "decoded values differ from qtip_quantize_tiles"
        gpu.linear.kernel_status()  # the status word kept in the built-in scratch is clean after each call


def test_noalloc_rejects_oversized_batch(gpu):
    lut_d, _ = gpu.codec.device_lut(gpu.synth.seeded_tlut(1))
    X = torch.zeros((65, 256), dtype=torch.float32, device="cuda")
    st = torch.zeros((65, 128), dtype=torch.int16, device="cuda")
    hat = torch.zeros((65, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(gpu.QtipError) as e:
        call_noalloc(gpu, X, lut_d, st, hat)
    assert e.value.code == -3 and "64" in str(e.value)


def test_noalloc_timeouts_are_reported_once(gpu):
    """A caller of this entry point holds no workspace, so a hand-shake that ran out is reported by
    qtip_kernel_status(), which also clears the word. The word is written from the host here: no kernel is made to
    wait."""
    lut_d, _ = gpu.codec.device_lut(gpu.synth.seeded_tlut(1))
    X = torch.zeros((4, 256), dtype=torch.float32, device="cuda")
    st = torch.zeros((4, 128), dtype=torch.int16, device="cuda")
    hat = torch.zeros((4, 256), dtype=torch.float32, device="cuda")
    call_noalloc(gpu, X, lut_d, st, hat)  # resolves the scratch address on this device
    gpu.linear.kernel_status()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for which in (0, 1, 2):  # tensor-core kernels, kernel-level cluster launches, built-in scratch
        gpu.lib().call("qtip_debug_set_status", which, 1, stream)
        with pytest.raises(gpu.QtipError) as e:
            gpu.linear.kernel_status()
        assert e.value.code == -5
        gpu.linear.kernel_status()  # cleared by the read: reported once
    # a later call does not clear a pending report by itself
    gpu.lib().call("qtip_debug_set_status", 2, 1, stream)
    call_noalloc(gpu, X, lut_d, st, hat)
    with pytest.raises(gpu.QtipError):
        gpu.linear.kernel_status()
    gpu.linear.kernel_status()
