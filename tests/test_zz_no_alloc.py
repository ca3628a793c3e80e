"""The decode-attention entry point that allocates nothing.

Some users of the library cannot allocate device memory where they call it: a
runtime that passes a custom call only its declared inputs and outputs, a
serving loop with a memory pool fixed at start-up, code that runs where
cudaMalloc is not allowed.  ``b200_attention_decode_static`` keeps its scratch
in a fixed array inside the library.  This test calls it twice in a row through
the C ABI and compares each result with ``b200_attention_decode`` (caller-owned
scratch) on the same inputs, and with an fp64 torch computation of the same
attention, so that a fault shared by both entry points cannot hide.  The two
entry points share their kernels, so their results must agree to the bit; the
comparisons use the tolerance of the other decode tests.  The file sorts last so
that a run that stops at the first failure has already run everything else.
"""
import gc
import math

import pytest
import torch

import b200_llama as B

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(batch, ctx, H, hs, dtype, page, seed):
    g = torch.Generator().manual_seed(seed)
    d = H * hs
    max_pages = (ctx + page - 1) // page
    n_pages = batch * max_pages + 2
    kv = torch.randn(2, n_pages, H, page, hs, generator=g).to(dtype).to(DEV)  # head-major pages
    q = torch.randn(batch, d, generator=g).to(dtype).to(DEV)
    table = torch.randperm(n_pages, generator=g)[: batch * max_pages].view(batch, max_pages).int().to(DEV)
    return q, kv, table


def _torch_reference(q, kv, table, ctx, H):
    """softmax(q K^T / sqrt(hs)) V per (sequence, head) over the first ctx rows the page table names, in fp64."""
    batch, d = q.shape
    hs = d // H
    page = kv.shape[3]
    rows = torch.arange(ctx, device=q.device)
    pg = table.long()[:, rows // page]                                   # [batch, ctx]
    off = (rows % page)[None, :].expand(batch, -1)
    k = kv[0][pg, :, off, :].double()                                    # [batch, ctx, H, hs]
    v = kv[1][pg, :, off, :].double()
    att = torch.einsum("bhe,buhe->bhu", q.double().view(batch, H, hs), k) / math.sqrt(hs)
    return torch.einsum("bhu,buhe->bhe", torch.softmax(att, -1), v).reshape(batch, d)


@pytest.mark.parametrize("batch,ctx,H,hs,dtype,page", [(2, 1000, 2, 64, torch.bfloat16, 64),
                                                       (64, 300, 8, 128, torch.bfloat16, 128),
                                                       (1, 40, 6, 48, torch.float32, 16)])
def test_static_scratch_matches_caller_scratch_twice(batch, ctx, H, hs, dtype, page):
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    for call in range(2):  # the second call reuses the array with the first call's contents in it
        q, kv, table = _case(batch, ctx + call, H, hs, dtype, page, seed=call)
        want = B.attention_decode(q, kv, table, ctx + call, H)
        out = torch.full_like(want, float("nan"))
        gc.collect()  # earlier tests' tensors must not be freed between the two readings
        mem_before = torch.cuda.memory_allocated()
        B.attention_decode_static(q, kv, table, ctx + call, H, out)
        assert torch.cuda.memory_allocated() <= mem_before  # the host layer allocates nothing either
        torch.cuda.synchronize()
        assert torch.allclose(out.float(), want.float(), rtol=tol, atol=tol)
        assert torch.equal(out, want)
        ref = _torch_reference(q, kv, table, ctx + call, H)
        assert torch.allclose(out.double(), ref, rtol=tol, atol=tol)


def test_static_scratch_rejects_problems_beyond_its_size():
    # 512 sequences x 32 heads x 130 floats = 2.1 M floats > the 1 M-float array
    q, kv, table = _case(512, 8, 32, 128, torch.bfloat16, 16, seed=3)
    out = torch.empty_like(q)
    with pytest.raises(B.B200Error) as e:
        B.attention_decode_static(q, kv, table, 8, 32, out)
    assert e.value.status == 5
    assert "built-in scratch" in str(e.value)
