"""Parity at the shapes of the benchmark configurations themselves.

The other GPU tests use small models; here each configuration is run at its own
dimensions against the CPU oracle (seeded synthetic weights and tokens of the
configuration's shapes and distributions):

* config 2: the full 12-layer 110M model, 2 sequences of 1024 tokens, bf16 against the fp32 oracle on the
  bf16-rounded weights, 2e-2 of the largest logit;
* config 3: the VJP of that model, 1 sequence of 1024 tokens, vocabulary 32000, against fp64 autograd, 3e-2 of
  each leaf's largest gradient;
* configs 4 and 5: a 2-layer slice of the 7B shape (dim 4096, hidden 11008, 32 heads of 128, vocabulary 32000):
  a 2048-token prefill, and decode steps at positions 4096.. over a paged cache of N(0,1) rows (33 pages of 128
  rows per sequence, rotation angles of positions beyond 4096).
"""
import math

import pytest
import torch

import b200_llama as B
from oracle import llama_ref as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bf16_weights(cfg, seed, gains_one=True):
    w = O.make_weights(cfg, seed, torch.float32, std=0.02, gains_one=gains_one)
    return {k: v.bfloat16() for k, v in w.items()}


def _plan(cfg, wb, with_t=False):
    p = B.Plan(cfg, torch.bfloat16)
    p.pack_weights({k: v.to(DEV).contiguous() for k, v in wb.items()}, with_transposed=with_t)
    return p


def _norm_rel(a, b):
    return float((a.double().cpu() - b.double()).abs().max() / b.double().abs().max())


def test_config2_full_model_forward():
    cfg = O.CONFIGS["c2"]
    wb = _bf16_weights(cfg, 21)
    tokens = O.make_tokens(cfg, 2, 1024, 22)
    with torch.no_grad():
        ref = O.forward_sequence(tokens, cfg, {k: v.float() for k, v in wb.items()})
    p = _plan(cfg, wb)
    got = p.forward(tokens.int().to(DEV))
    torch.cuda.synchronize()
    assert B.device_status() == 0
    assert _norm_rel(got, ref) < 2e-2  # bf16 bar: 2e-2 of the fp32 reference, normalised by the largest logit
    # next-token choice: equal wherever the oracle's top-2 gap is wider than the bf16 bar
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 2 * 2e-2 * ref.abs().max()
    if clear.any():
        assert torch.equal(got.cpu().argmax(-1)[clear], ref.argmax(-1)[clear])
    p.close()


def test_config3_full_model_vjp():
    """12 layers, vocabulary 32000, 1024 tokens: the classifier-gradient GEMM (32000 x 768 over 1024 tokens) and the
    K = 1024 weight-gradient GEMMs run at their benchmark widths."""
    cfg = O.CONFIGS["c2"]
    wb = _bf16_weights(cfg, 23, gains_one=False)
    tokens = O.make_tokens(cfg, 1, 1024, 24)
    g = torch.Generator().manual_seed(25)
    dlogits = torch.randn(1, 1024, cfg["vocab_size"], generator=g)  # cotangent ~N(0,1) fp32
    ref_logits, ref = O.vjp_sequence(tokens, cfg, {k: v.double() for k, v in wb.items()}, dlogits.double())
    p = _plan(cfg, wb, with_t=True)
    tok = tokens.int().to(DEV)
    saved = p.new_saved(1, 1024)
    logits = p.forward(tok, saved=saved)
    grads = p.backward(tok, dlogits.to(DEV).contiguous(), saved, p.new_grads())
    torch.cuda.synchronize()
    assert B.device_status() == 0
    assert _norm_rel(logits, ref_logits) < 2e-2
    leaves = p.unpack_grads(grads)
    for k, r in ref.items():
        err = float((leaves[k].double().cpu() - r).abs().max() / r.abs().max())
        assert err < 3e-2, (k, err)
    p.close()


SLICE_7B = dict(O.CONFIGS["c4"], n_layers=2, seq_len=4352)


def test_config4_slice_prefill():
    cfg = SLICE_7B
    wb = _bf16_weights(cfg, 26)
    tokens = O.make_tokens(cfg, 1, 2048, 27)
    with torch.no_grad():
        ref = O.forward_sequence(tokens, cfg, {k: v.float() for k, v in wb.items()})
    p = _plan(cfg, wb)
    got = p.forward(tokens.int().to(DEV))
    torch.cuda.synchronize()
    assert B.device_status() == 0
    assert _norm_rel(got, ref) < 2e-2
    p.close()


def test_config5_slice_decode_beyond_position_4096():
    cfg = SLICE_7B
    L, d, H = cfg["n_layers"], cfg["dim"], cfg["n_heads"]
    hs = d // H
    batch, ctx0, steps, page = 2, 4096, 3, 128
    wb = _bf16_weights(cfg, 28)
    wf = {k: v.float() for k, v in wb.items()}
    g = torch.Generator().manual_seed(29)
    # the cache rows the benchmark pre-fills: N(0,1), rounded to bf16 (scaled keys keep the softmax from being flat)
    past_k = (torch.randn(L, batch, ctx0, d, generator=g) * 2.0).bfloat16()
    past_v = torch.randn(L, batch, ctx0, d, generator=g).bfloat16()
    tokens = O.make_tokens(cfg, batch, steps, 30)

    p = _plan(cfg, wb)
    max_pages = (ctx0 + steps + page - 1) // page  # 33
    assert max_pages == 33
    n_pages = batch * max_pages + 3
    kv = p.new_kv_pages(n_pages, page)
    perm = torch.randperm(n_pages, generator=g)[: batch * max_pages]
    table = perm.view(batch, max_pages).int().to(DEV)
    # [L, B, ctx, d] -> head-major pages [L, 2, page, H, row, hs]
    rows = torch.arange(ctx0)
    pg = table.cpu().long()[:, rows // page]          # [B, ctx]
    off = (rows % page)[None, :].expand(batch, -1)    # [B, ctx]
    for part, past in ((0, past_k), (1, past_v)):
        src = past.view(L, batch, ctx0, H, hs).to(DEV)
        for l in range(L):
            # kv[l, part] is [n_pages, H, page, hs]; index (page, row) pairs, heads stay in the middle
            kv[l, part][pg.reshape(-1).to(DEV), :, off.reshape(-1).to(DEV), :] = src[l].reshape(batch * ctx0, H, hs)

    pk, pv = past_k.float(), past_v.float()
    tok = tokens.int().to(DEV)
    for i in range(steps):
        with torch.no_grad():
            ref, aux = O.forward_sequence(tokens[:, i:i + 1], cfg, wf, past_k=pk, past_v=pv, return_aux=True)
        _, logits = p.decode_step(ctx0 + i, kv, table, tokens=tok[:, i].contiguous())
        torch.cuda.synchronize()
        assert _norm_rel(logits, ref[:, 0]) < 2e-2, i
        # the appended cache row of every layer against the oracle's rotated key (angle of position 4096 + i)
        pgi = table.cpu().long()[:, (ctx0 + i) // page]
        for l in range(L):
            got_k = kv[l, 0][pgi.to(DEV), :, (ctx0 + i) % page, :].reshape(batch, d).float().cpu()
            want_k = aux["k"][l][:, 0]
            assert float((got_k - want_k).abs().max() / want_k.abs().max()) < 2e-2, (i, l)
        # the oracle's context grows by the rows it produced itself (bf16-rounded, as the cache stores them)
        pk = torch.cat([pk, aux["k"].bfloat16().float()], dim=2)
        pv = torch.cat([pv, aux["v"].bfloat16().float()], dim=2)
    assert B.device_status() == 0
    p.close()


@pytest.mark.parametrize("M,N,K", [(512, 4096, 4096), (256, 4096, 11008), (64, 4096, 11008), (64, 12288, 4096),
                                   (2048, 1536, 4096), (2048, 4096, 1376)])
def test_gemm_exact_at_7b_depths(M, N, K):
    """K = 4096 and 11008 (and the per-rank K = 11008/8 of tensor parallelism): integer operands in [-2, 2] keep
    every partial sum exact in fp32, so the result must equal the reference bit for bit."""
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randint(-2, 3, (M, K), generator=g).bfloat16().to(DEV)
    b = torch.randint(-2, 3, (N, K), generator=g).bfloat16().to(DEV)
    y = B.gemm(a, b, out_dtype=torch.float32, impl=1)
    assert B.device_status() == 0
    assert torch.equal(y, a.float() @ b.float().T)


def test_rope_table_positions_beyond_4096():
    """Rotation of the projection's output at positions 4096..4223 (the decode positions of config 5) against
    fp64 angles: a plan with seq_len 4224 and a one-layer model whose q/k projection is the identity."""
    hs, H = 128, 2
    d = H * hs
    cfg = dict(dim=d, hidden_dim=256, n_layers=1, n_heads=H, n_kv_heads=H, vocab_size=256, seq_len=4224)
    w = O.make_weights(cfg, 31, torch.float32, std=0.05)
    eye = torch.eye(d)
    w["wq"][0], w["wk"][0] = eye.clone(), eye.clone()
    wb = {k: v.bfloat16() for k, v in w.items()}
    p = _plan(cfg, wb)
    batch, page = 1, 128
    pos = 4200
    kv = p.new_kv_pages(33, page)
    table = torch.arange(33, dtype=torch.int32, device=DEV).view(1, 33)
    tok = torch.tensor([7], dtype=torch.int32, device=DEV)
    p.decode_step(pos, kv, table, tokens=tok, want_logits=False, want_hidden=True)
    torch.cuda.synchronize()
    x = wb["token_embedding_table"][7].double()
    xb = (x * torch.rsqrt((x * x).mean() + 1e-5)).bfloat16().double()  # the projection's bf16 operand
    j2 = torch.arange(0, hs, 2, dtype=torch.float64)
    ang = pos / torch.pow(torch.tensor(10000.0, dtype=torch.float64), j2 / hs)
    c, s = torch.cos(ang).repeat(H), torch.sin(ang).repeat(H)
    want = torch.stack((c * xb[0::2] - s * xb[1::2], s * xb[0::2] + c * xb[1::2]), -1).flatten()
    got = kv[0, 0, pos // page, :, pos % page, :].reshape(d).double().cpu()
    assert float((got - want).abs().max() / want.abs().max()) < 8e-3  # one bf16 rounding of the stored row
    assert B.device_status() == 0
    p.close()
