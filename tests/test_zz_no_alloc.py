"""The allocation-free entry point (vx_blkscale_gemm_noalloc) against the regular route.

Some hosts cannot call cudaMalloc once they are running: a serving worker that has handed the
whole device to its own memory pool, or an audio thread with a latency budget (an allocation
may stall every stream while the driver synchronises).  For them the library keeps the
tensor-core copy of the block scales in a fixed array of its own.  This test calls that entry
point straight through the C ABI, twice in a row with different problems, and requires the
same bytes as ``dgx_mxfp4_blkscale_gemm`` (which allocates its scratch through torch).  The
second call reuses the array the first one filled, so stale contents would show up here.

Collected last on purpose (file name): a run that stops at the first failure has by then
executed every other test.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, aq, bq, asc, bsc, M, N, K):
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    rc = lib.vx_blkscale_gemm_noalloc(aq.data_ptr(), bq.data_ptr(), asc.data_ptr(), bsc.data_ptr(), out.data_ptr(),
                                      M, N, K, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.vx_last_error().decode()
    return out


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    from velox_voice_b200 import _lib, ops

    lib = _lib.load()
    torch.manual_seed(11)
    for M, N, K in [(300, 200, 512), (130, 136, 1024)]:  # second problem is smaller in M: stale rows would leak
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = torch.randn(N, K, device="cuda").bfloat16()
        aq, asc = ops.mxfp4_block_quantize(x, mode="A")
        bq, bsc = ops.mxfp4_block_quantize(w, mode="B")
        want = ops.dgx_mxfp4_blkscale_gemm(aq, bq, asc, bsc)
        got = _call_noalloc(lib, aq, bq, asc, bsc, M, N, K)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"{M}x{N}x{K}: max |diff| = {(got - want).abs().max().item()}"
    assert _lib.device_status() == 0


def test_noalloc_rejects_oversized_problems_before_launching():
    from velox_voice_b200 import _lib

    lib = _lib.load()
    M, N, K = 131072, 128, 512  # A-side scale factors need 4 MiB > the 2 MiB built-in scratch
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = lib.vx_blkscale_gemm_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                      dummy.data_ptr(), M, N, K, None)
    assert rc < 0
    assert b"too large" in lib.vx_last_error()
    assert lib.vx_blkscale_gemm_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                        dummy.data_ptr(), 3, 128, 512, None) < 0  # odd M
