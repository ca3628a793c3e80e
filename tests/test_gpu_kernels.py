"""Single kernels through the C ABI against torch fp32/fp64 references."""
import math

import pytest
import torch

import b200_llama as B

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def _ints(shape, seed, lo=-2, hi=3, dtype=torch.bfloat16):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(lo, hi, shape, generator=g).to(dtype).to(DEV)


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (256, 512, 768), (384, 768, 2048),
                                   (100, 96, 72), (8192, 2304, 768), (64, 4096, 1024), (1, 32, 8),
                                   # large enough for the CTA-pair kernel (256-row tiles), with M and K tails
                                   (4096, 768, 2048), (8192, 1024, 256), (5000, 1536, 704), (8192, 32000, 64),
                                   # 192-column pair tiles (N = 768, 1152), with an M tail
                                   (8192, 768, 512), (8000, 1152, 192),
                                   # widths that no tile width divides (per-rank widths of 8-way tensor parallelism:
                                   # 2 x 11008 / 8 = 2752, 32000 / 8 = 4000): a partly filled last column of tiles
                                   (8192, 2752, 256), (4096, 4000, 128), (8192, 1376, 192), (8192, 2720, 64)])
def test_gemm_bf16_exact_on_small_integers(impl, M, N, K):
    # integer operands in [-2,2]: every product and partial sum is exact in fp32
    a, b = _ints((M, K), 1), _ints((N, K), 2)
    y = B.gemm(a, b, out_dtype=torch.float32, impl=impl)
    ref = a.float() @ b.float().T
    assert B.device_status() == 0
    assert torch.equal(y, ref)


@pytest.mark.parametrize("M,N", [(8192, 768), (8192, 1024), (8000, 1152), (8192, 640), (8192, 2752), (8192, 1472)])
def test_pair_gemm_bf16_output_exact(M, N):
    # K = 64 and operands in [-2,2]: |sums| <= 256, exact in bf16, so the staged bf16 store path is checked bit for bit
    a, b = _ints((M, 64), 3), _ints((N, 64), 4)
    y = B.gemm(a, b, out_dtype=torch.bfloat16, impl=1)
    assert B.device_status() == 0
    assert torch.equal(y.float(), a.float() @ b.float().T)


@pytest.mark.parametrize("impl", [1, 2])
def test_gemm_bf16_random_and_bf16_out(impl):
    g = torch.Generator().manual_seed(0)
    a = torch.randn(512, 768, generator=g).bfloat16().to(DEV)
    b = (torch.randn(1024, 768, generator=g) * 0.02).bfloat16().to(DEV)
    ref = a.double() @ b.double().T
    y32 = B.gemm(a, b, out_dtype=torch.float32, impl=impl)
    assert _rel(y32, ref) < 1e-5
    y16 = B.gemm(a, b, out_dtype=torch.bfloat16, impl=impl)
    assert _rel(y16, ref) < 6e-3
    assert B.device_status() == 0


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(200, 144, 136),      # few tiles: the 32-row form of the FFMA kernel, ragged edges
                                   (2312, 1088, 72)])    # 19 x 17 tiles: its 128-row form
def test_gemm_transposed_operands(ta, tb, dtype, M, N, K):
    a = _ints((K, M) if ta else (M, K), 3, dtype=dtype)
    b = _ints((K, N) if tb else (N, K), 4, dtype=dtype)
    y = B.gemm(a, b, ta=ta, tb=tb, out_dtype=torch.float32 if dtype == torch.float32 else torch.float32)
    ref = (a.float().T if ta else a.float()) @ (b.float() if tb else b.float().T)
    assert torch.equal(y, ref)
    y2 = B.gemm(a, b, ta=ta, tb=tb, out=y.clone(), accumulate=True)
    assert torch.equal(y2, 2 * ref)


def test_gemm_fp32_matches_fp64_reference():
    g = torch.Generator().manual_seed(5)
    a = torch.randn(256, 288, generator=g).to(DEV)
    b = (torch.randn(864, 288, generator=g) * 0.02).to(DEV)
    y = B.gemm(a, b)
    ref = a.double() @ b.double().T
    assert torch.allclose(y.double(), ref, rtol=1e-5, atol=1e-6)


def test_gemm_is_deterministic():
    a, b = torch.randn(1024, 768, device=DEV).bfloat16(), torch.randn(768, 768, device=DEV).bfloat16()
    y0 = B.gemm(a, b, out_dtype=torch.float32)
    for _ in range(3):
        assert torch.equal(B.gemm(a, b, out_dtype=torch.float32), y0)


def test_gemm_rejects_bad_arguments():
    a = torch.zeros(16, 16, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(B.B200Error) as e:
        B.gemm(a, torch.zeros(8, 16, device=DEV, dtype=torch.bfloat16))  # N not a multiple of 16
    assert e.value.status == 2
    with pytest.raises(B.B200Error):
        B.gemm(a.float(), a.float(), impl=1)  # the tensor-core kernel is bf16 only


@pytest.mark.parametrize("rows,dim", [(7, 64), (256, 288), (1000, 768), (64, 4096)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(rows, dim, out_dtype):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(rows, dim, generator=g).to(DEV)
    gain = (1 + 0.1 * torch.randn(dim, generator=g)).to(DEV)
    y, rinv = B.rmsnorm(x, gain, 1e-5, out_dtype)
    r = torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5)
    ref = gain.double() * x.double() * r
    tol = 1e-5 if out_dtype == torch.float32 else 8e-3
    assert torch.allclose(y.double(), ref, rtol=tol, atol=tol)
    assert torch.allclose(rinv.double(), r[:, 0], rtol=1e-5)


def _attn_ref(q, k, v, B_, S, H):
    hs = q.shape[1] // H
    q, k, v = (t.double().view(B_, S, H, hs).transpose(1, 2) for t in (q, k, v))
    att = q @ k.transpose(-1, -2) / math.sqrt(hs)
    att = att.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    lse = torch.logsumexp(att, -1)
    o = torch.softmax(att, -1) @ v
    return o.transpose(1, 2).reshape(B_ * S, H * hs), lse


@pytest.mark.parametrize("impl", [0, 2])
@pytest.mark.parametrize("B_,S,H,hs,dtype", [(1, 256, 6, 48, torch.float32), (2, 100, 2, 32, torch.float32),
                                             (2, 256, 4, 64, torch.bfloat16), (1, 384, 2, 128, torch.bfloat16),
                                             (3, 33, 2, 16, torch.bfloat16), (2, 200, 3, 64, torch.bfloat16),
                                             (2, 1024, 2, 64, torch.bfloat16), (2, 300, 2, 128, torch.bfloat16)])
def test_attention_forward(impl, B_, S, H, hs, dtype):
    g = torch.Generator().manual_seed(2)
    qkv = torch.randn(B_ * S, 3 * H * hs, generator=g).to(dtype).to(DEV)
    d = H * hs
    q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
    o, lse = B.attention(q, k, v, B_, S, H, impl=impl)
    ro, rl = _attn_ref(q, k, v, B_, S, H)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(o.double(), ro, rtol=tol, atol=tol)
    assert torch.allclose(lse.double(), rl, rtol=1e-4, atol=1e-4 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("B_,S,H,gain", [(2, 384, 2, 1.0), (1, 640, 3, 3.0), (2, 1024, 2, 3.0), (3, 130, 2, 2.0)])
def test_attention_forward_tensor_core_edges(B_, S, H, gain):
    """Tensor-core kernel, output accumulated in tensor memory: an odd number of tiles, a ragged tail, and scores
    spread widely enough (gain > 1) that block maxima exceed the running reference by more than 2^8, so that the
    in-place rescale of the accumulator runs."""
    g = torch.Generator().manual_seed(7)
    d = H * 64
    qkv = (torch.randn(B_ * S, 3 * d, generator=g) * gain).bfloat16().to(DEV)
    q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
    o, lse = B.attention(q, k, v, B_, S, H, impl=1)
    assert B.device_status() == 0
    ro, rl = _attn_ref(q, k, v, B_, S, H)
    assert torch.allclose(o.double(), ro, rtol=1e-2, atol=1e-2 * gain)
    assert torch.allclose(lse.double(), rl, rtol=1e-4, atol=2e-2)


def _decode_case(batch, ctx, H, hs, dtype, page, seed=0):
    g = torch.Generator().manual_seed(seed)
    d = H * hs
    max_pages = (ctx + page - 1) // page
    n_pages = batch * max_pages + 3
    kv = torch.randn(2, n_pages, H, page, hs, generator=g).to(dtype).to(DEV)  # head-major pages
    q = torch.randn(batch, d, generator=g).to(dtype).to(DEV)
    table = torch.randperm(n_pages, generator=g)[: batch * max_pages].view(batch, max_pages).int().to(DEV)
    return q, kv, table


def _decode_ref(q, kv, table, ctx, H):
    batch, d = q.shape
    hs = d // H
    page = kv.shape[3]
    out = torch.empty(batch, d, dtype=torch.float64)
    for b in range(batch):
        rows = [(int(table[b, u // page]), u % page) for u in range(ctx)]
        k = torch.stack([kv[0, p, :, r] for p, r in rows]).double().cpu()  # [ctx, H, hs]
        v = torch.stack([kv[1, p, :, r] for p, r in rows]).double().cpu()
        qq = q[b].double().cpu().view(H, hs)
        att = torch.softmax(torch.einsum("he,uhe->hu", qq, k) / math.sqrt(hs), -1)
        out[b] = torch.einsum("hu,uhe->he", att, v).reshape(d)
    return out


@pytest.mark.parametrize("batch,ctx,H,hs,dtype,page", [(1, 6, 6, 48, torch.float32, 16), (2, 700, 2, 64, torch.bfloat16, 64),
                                                       (3, 333, 4, 128, torch.bfloat16, 32), (64, 130, 8, 128, torch.bfloat16, 128)])
def test_attention_decode_paged(batch, ctx, H, hs, dtype, page):
    q, kv, table = _decode_case(batch, ctx, H, hs, dtype, page)
    o = B.attention_decode(q, kv, table, ctx, H)
    ref = _decode_ref(q, kv, table, ctx, H)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(o.double().cpu(), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("ta,tb", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 192), (2304, 768, 1024), (200, 144, 136)])
def test_gemm_tensor_core_transposed_operands(ta, tb, M, N, K):
    a = _ints((K, M) if ta else (M, K), 3)
    b = _ints((K, N) if tb else (N, K), 4)
    y = B.gemm(a, b, ta=ta, tb=tb, out_dtype=torch.float32, impl=1)
    ref = (a.float().T if ta else a.float()) @ (b.float() if tb else b.float().T)
    assert B.device_status() == 0
    assert torch.equal(y, ref)


@pytest.mark.parametrize("impl", [0, 2])
@pytest.mark.parametrize("B_,S,H,hs,dtype", [(2, 256, 3, 64, torch.bfloat16), (1, 200, 2, 64, torch.bfloat16),
                                             (2, 1024, 2, 64, torch.bfloat16), (1, 96, 2, 48, torch.float32)])
def test_attention_backward(impl, B_, S, H, hs, dtype):
    g = torch.Generator().manual_seed(5)
    d = H * hs
    qkv = torch.randn(B_ * S, 3 * d, generator=g).to(dtype).to(DEV)
    d_o = torch.randn(B_ * S, d, generator=g).to(dtype).to(DEV)
    ref_in = qkv.double().clone().requires_grad_(True)
    ro, _ = _attn_ref(ref_in[:, :d], ref_in[:, d:2 * d], ref_in[:, 2 * d:], B_, S, H)
    ro.backward(d_o.double())
    o, lse = B.attention(qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:], B_, S, H, impl=impl)
    dqkv = B.attention_backward(qkv, o, lse, d_o, B_, S, H, impl=impl)
    assert B.device_status() == 0
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for name, sl in (("dq", slice(0, d)), ("dk", slice(d, 2 * d)), ("dv", slice(2 * d, 3 * d))):
        r = ref_in.grad[:, sl]
        err = float((dqkv[:, sl].double() - r).abs().max() / r.abs().max())
        assert err < tol, (name, err)
