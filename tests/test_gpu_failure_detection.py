"""Bounded device-side waits: a wait that nothing satisfies runs out, the kernel returns, the status
word reports it, and the context stays usable.  No GPU fault, trap or hang is involved."""
import ctypes

import pytest
import torch

import b200_llama as B

pytestmark = pytest.mark.gpu


def test_unsatisfied_wait_times_out_and_reports_status():
    assert B.device_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    # 40 M cycles: about 20 ms at 1.9 GHz
    B.check(B.lib().b200_selftest_bounded_wait(40_000_000, flag.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(flag.item()) == 1          # the kernel ran to its end after giving up
    with pytest.raises(B.B200Error) as e:
        B.device_status()
    assert e.value.status == 9            # B200_ERR_TIMEOUT
    assert B.device_status() == 0         # reading the word cleared it
    # the context is intact: a tensor-core GEMM still runs and is exact
    a = torch.randint(-2, 3, (256, 128)).bfloat16().cuda()
    b = torch.randint(-2, 3, (128, 128)).bfloat16().cuda()
    y = B.gemm(a, b, out_dtype=torch.float32, impl=1)
    assert torch.equal(y, a.float() @ b.float().T)
    assert B.device_status() == 0


def test_selftest_rejects_unbounded_budgets():
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert B.lib().b200_selftest_bounded_wait(0, flag.data_ptr(), None) == 1
    assert B.lib().b200_selftest_bounded_wait(10**12, flag.data_ptr(), None) == 1


def test_unanswered_peer_wait_times_out_and_reports_status():
    """The wait that tensor-parallel kernels perform on other ranks' flags, on one GPU: nothing sets the flags, the
    budget (about 20 ms) runs out, the kernel returns, the status word says so, the context stays usable."""
    assert B.device_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    B.check(B.lib().b200_selftest_peer_wait(40_000_000, flag.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    with pytest.raises(B.B200Error) as e:
        B.device_status()
    assert e.value.status == 9 and "0x1000" in str(e.value)   # ST_PEER_TIMEOUT
    assert B.device_status() == 0
    x = torch.randn(64, 256, device="cuda")
    y, _ = B.rmsnorm(x, torch.ones(256, device="cuda"))
    assert torch.allclose(y, x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5), rtol=1e-5, atol=1e-6)
    assert B.lib().b200_selftest_peer_wait(0, flag.data_ptr(), None) == 1
