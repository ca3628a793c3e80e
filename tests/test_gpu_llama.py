"""The llama forward / VJP / decode path through the C ABI against the CPU oracle."""
import numpy as np
import pytest
import torch

import b200_llama as B
from oracle import llama_ref as O

pytestmark = pytest.mark.gpu
DEV = "cuda"

SMALL = dict(dim=128, hidden_dim=256, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=512, seq_len=64)


def _to_dev(w, dtype):
    return {k: v.to(dtype).to(DEV).contiguous() for k, v in w.items()}


def _plan(cfg, w, dtype, with_t=False):
    p = B.Plan(cfg, dtype)
    p.pack_weights(_to_dev(w, dtype), with_transposed=with_t)
    return p


def _norm_rel(a, b):
    return float((a.double().cpu() - b.double()).abs().max() / b.double().abs().max())


@pytest.mark.parametrize("name,batch,seq", [("tiny", 2, 16), ("small", 2, 64), ("c1", 1, 256)])
def test_forward_fp32_matches_oracle(name, batch, seq):
    cfg = SMALL if name == "small" else O.CONFIGS[name]
    w = O.make_weights(cfg, 3, torch.float32, std=0.02 if name == "c1" else 0.1, gains_one=(name == "c1"))
    tokens = O.make_tokens(cfg, batch, seq, 1)
    ref = O.forward_sequence(tokens, cfg, O.cast_weights(w, torch.float64))
    p = _plan(cfg, w, torch.float32)
    got = p.forward(tokens.int().to(DEV))
    torch.cuda.synchronize()
    assert B.device_status() == 0
    # fp32 bar: 1e-4 relative, 1e-5 absolute
    assert torch.allclose(got.double().cpu(), ref, rtol=1e-4, atol=1e-5)
    # argmax tokens bit-exact wherever the top-2 gap is above the fp32 bar
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 1e-4 * top2[..., 0].abs() + 1e-5
    assert clear.float().mean() > 0.9
    assert torch.equal(got.cpu().argmax(-1)[clear], ref.argmax(-1)[clear])


def test_forward_fp32_against_golden_hidden():
    """Golden vectors come from the reference's own forward source (tests/golden/make_golden.py)."""
    import os
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "llama_golden.npz"))["D_hidden_f64"]
    cfg = O.CONFIGS["tiny"]
    w = O.make_weights(cfg, 5, torch.float64, std=0.2, gains_one=False)
    tokens = O.make_tokens(cfg, 2, 12, 3)
    p = _plan(cfg, w, torch.float32)
    logits = p.forward(tokens.int().to(DEV)).double().cpu()
    ref_logits = torch.from_numpy(gold) @ w["wcls"].T
    assert torch.allclose(logits, ref_logits, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("gemm_impl", ["0", "2"])
@pytest.mark.parametrize("name,batch,seq", [("small", 2, 64), ("c2mini", 2, 256)])
def test_forward_bf16_within_2e2_of_fp32_oracle(monkeypatch, gemm_impl, name, batch, seq):
    monkeypatch.setenv("B200_GEMM_IMPL", gemm_impl)
    cfg = SMALL if name == "small" else dict(O.CONFIGS["c2"], n_layers=2, seq_len=256)
    w = O.make_weights(cfg, 4, torch.float32)
    wb = {k: v.bfloat16() for k, v in w.items()}
    tokens = O.make_tokens(cfg, batch, seq, 2)
    # the oracle runs in fp32 on the bf16-rounded weights (the model the GPU sees)
    ref = O.forward_sequence(tokens, cfg, {k: v.float() for k, v in wb.items()})
    p = _plan(cfg, wb, torch.bfloat16)
    got = p.forward(tokens.int().to(DEV))
    torch.cuda.synchronize()
    assert B.device_status() == 0
    assert _norm_rel(got, ref) < 2e-2


def test_forward_keeps_activations_and_kv(monkeypatch):
    cfg = SMALL
    w = O.make_weights(cfg, 6, torch.float32, std=0.1)
    tokens = O.make_tokens(cfg, 2, 32, 5)
    ref, aux = O.forward_sequence(tokens, cfg, O.cast_weights(w, torch.float64), return_aux=True)
    p = _plan(cfg, w, torch.float32)
    saved = p.new_saved(2, 32)
    kv = torch.empty(cfg["n_layers"], 2, 2, 32, cfg["dim"], device=DEV)
    got = p.forward(tokens.int().to(DEV), saved=saved, kv_out=kv)
    assert torch.allclose(got.double().cpu(), ref, rtol=1e-4, atol=1e-5)
    assert torch.allclose(kv[:, 0].double().cpu(), aux["k"], rtol=1e-4, atol=1e-5)
    assert torch.allclose(kv[:, 1].double().cpu(), aux["v"], rtol=1e-4, atol=1e-5)


def _grad_check(cfg, dtype, batch, seq, rtol, std):
    w = O.make_weights(cfg, 7, torch.float32, std=std, gains_one=False)
    wq = {k: v.to(dtype) for k, v in w.items()}
    tokens = O.make_tokens(cfg, batch, seq, 9)
    g = torch.Generator().manual_seed(11)
    dlogits = torch.randn(batch, seq, cfg["vocab_size"], generator=g)
    _, ref = O.vjp_sequence(tokens, cfg, {k: v.double() for k, v in wq.items()}, dlogits.double())
    p = _plan(cfg, wq, dtype, with_t=True)
    saved = p.new_saved(batch, seq)
    tok = tokens.int().to(DEV)
    p.forward(tok, saved=saved)
    grads = p.new_grads()
    p.backward(tok, dlogits.to(DEV).contiguous(), saved, grads)
    torch.cuda.synchronize()
    assert B.device_status() == 0
    leaves = p.unpack_grads(grads)
    for k, r in ref.items():
        got = leaves[k].double().cpu()
        err = float((got - r).abs().max() / r.abs().max())
        assert err < rtol, (k, err)
        if dtype == torch.float32:
            # the fp32 bar element by element: 1e-4 relative, with the absolute floor of 1e-5 scaled to the leaf
            # (gradients of a sum over 64 tokens x 512 logits have magnitudes far from 1)
            assert torch.allclose(got, r, rtol=1e-4, atol=1e-5 * float(r.abs().max().clamp_min(1.0))), k
    return p, tok, dlogits, saved, leaves


def test_vjp_fp32_matches_oracle():
    _grad_check(SMALL, torch.float32, 2, 32, 1e-4, 0.1)


def test_vjp_bf16_close_to_oracle_and_accumulates():
    p, tok, dlogits, saved, leaves = _grad_check(SMALL, torch.bfloat16, 2, 32, 3e-2, 0.1)
    grads = p.new_grads()
    dl = dlogits.to(DEV).contiguous()
    p.backward(tok, dl, saved, grads)
    p.backward(tok, dl, saved, grads, accumulate=True)
    twice = p.unpack_grads(grads)
    for k in leaves:
        assert torch.allclose(twice[k], 2 * leaves[k], rtol=1e-5, atol=1e-6), k


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_steps_match_full_forward(dtype):
    cfg = SMALL
    w = O.make_weights(cfg, 8, torch.float32, std=0.1)
    wq = {k: v.to(dtype) for k, v in w.items()}
    batch, seq, page = 3, 40, 16
    tokens = O.make_tokens(cfg, batch, seq, 6)
    ref = O.forward_sequence(tokens, cfg, {k: v.double() for k, v in wq.items()})
    p = _plan(cfg, wq, dtype)
    max_pages = (seq + page - 1) // page
    kv = p.new_kv_pages(batch * max_pages, page)
    # scatter the pages so that the table is exercised
    perm = torch.randperm(batch * max_pages, generator=torch.Generator().manual_seed(0))
    table = perm.view(batch, max_pages).int().to(DEV)
    tok = tokens.int().to(DEV)
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else None
    for pos in range(seq):
        _, logits = p.decode_step(pos, kv, table, tokens=tok[:, pos].contiguous())
        if tol:
            assert torch.allclose(logits.double().cpu(), ref[:, pos], **tol), pos
        else:
            assert _norm_rel(logits, ref[:, pos]) < 2e-2, pos
    assert B.device_status() == 0


def test_decode_reference_signature_hidden_state():
    """The reference's own call shape: one residual vector, a cache of `pos` rows, hidden state out."""
    cfg = O.CONFIGS["c1"]
    w = O.make_weights(cfg, 12, torch.float32, std=0.05)
    wn = O.to_numpy({k: v.double() for k, v in w.items()})
    rng = np.random.default_rng(3)
    pos = 5
    x = rng.standard_normal(cfg["dim"])
    kc = rng.standard_normal((cfg["n_layers"], pos, cfg["dim"]))
    vc = rng.standard_normal((cfg["n_layers"], pos, cfg["dim"]))
    ref = O.forward_token(x, cfg, wn, kc, vc)
    p = _plan(cfg, w, torch.float32)
    kv = p.new_kv_pages(1, 16)
    L, H = cfg["n_layers"], cfg["n_heads"]
    hs = cfg["dim"] // H
    # the reference's [L, pos, kv_dim] cache into head-major pages [L, 2, page, H, row, hs]
    kv[:, 0, 0, :, :pos] = torch.from_numpy(kc).float().view(L, pos, H, hs).permute(0, 2, 1, 3).to(DEV)
    kv[:, 1, 0, :, :pos] = torch.from_numpy(vc).float().view(L, pos, H, hs).permute(0, 2, 1, 3).to(DEV)
    table = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    hidden, _ = p.decode_step(pos, kv, table, x=torch.from_numpy(x).float().to(DEV).view(1, -1), want_hidden=True,
                              want_logits=False)
    assert torch.allclose(hidden[0].double().cpu(), torch.from_numpy(ref), rtol=1e-4, atol=1e-5)


def test_bad_calls_return_status_codes():
    cfg = SMALL
    p = B.Plan(cfg, torch.float32)
    with pytest.raises(B.B200Error) as e:
        B.Plan(dict(cfg, n_kv_heads=2), torch.float32)
    assert e.value.status == 10
    with pytest.raises(B.B200Error) as e:
        B.Plan(dict(cfg, dim=100), torch.float32)
    assert e.value.status == 2
    p.pack_weights(_to_dev(O.make_weights(cfg, 1), torch.float32))
    with pytest.raises(B.B200Error) as e:
        p.forward(torch.zeros(1, 1000, dtype=torch.int32, device=DEV))  # longer than seq_len
    assert e.value.status == 2
    tok = torch.zeros(1, 8, dtype=torch.int32, device=DEV)
    logits = torch.empty(1, 8, cfg["vocab_size"], device=DEV)
    ws = torch.empty(1024, dtype=torch.uint8, device=DEV)
    st = B.lib().b200_forward(p._h, tok.data_ptr(), 1, 8, p.packed.data_ptr(), logits.data_ptr(), None, None,
                              ws.data_ptr(), ws.numel(), None)
    assert st == 5  # workspace too small, nothing launched


def test_captured_graphs_replay_the_eager_forward():
    """capture_forward / capture_prefill_step: a replay gives the eager result bit for bit, and the captured
    step moves its tokens up from and its last-position logits down to pinned host memory."""
    cfg = SMALL
    w = O.make_weights(cfg, 5, torch.float32, std=0.1, gains_one=False)
    p = _plan(cfg, w, torch.bfloat16)
    t1, t2 = O.make_tokens(cfg, 4, 64, 1).int(), O.make_tokens(cfg, 4, 64, 2).int()
    eager1, eager2 = p.forward(t1.to(DEV)).clone(), p.forward(t2.to(DEV)).clone()
    tok = t1.to(DEV)
    logits = torch.empty_like(eager1)
    g = p.capture_forward(tok, logits)
    logits.zero_()
    g.replay()
    assert torch.equal(logits, eager1)
    host_tok = t2.clone().pin_memory()
    last, host_last = torch.empty(4, cfg["vocab_size"], device=DEV), torch.empty(4, cfg["vocab_size"]).pin_memory()
    gs = p.capture_prefill_step(host_tok, tok, logits, last, host_last)
    host_last.zero_()
    gs.replay()
    torch.cuda.synchronize()
    assert torch.equal(logits, eager2)
    assert torch.equal(host_last, eager2[:, -1, :].cpu())
    host_tok.copy_(t1)  # the graph reads the pinned buffer at replay time
    gs.replay()
    torch.cuda.synchronize()
    assert torch.equal(host_last, eager1[:, -1, :].cpu())
    with pytest.raises(B.B200Error):
        p.capture_prefill_step(t2, tok, logits, last, host_last)  # pageable host tokens
    assert B.device_status() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2)])
def test_forward_mode_matches_oracle(dtype, tol):
    """JVP with respect to every weight leaf (the `Forward` row of the reference's harness) against torch forward-mode
    AD in fp64; also with a tangent on a single leaf (the others absent count as zero)."""
    cfg = SMALL
    w = O.make_weights(cfg, 7, torch.float32, std=0.1, gains_one=False)
    wq = {k: v.to(dtype) for k, v in w.items()}
    g = torch.Generator().manual_seed(13)
    dw = {k: (0.1 * torch.randn(v.shape, generator=g)).to(dtype) for k, v in w.items()}
    tokens = O.make_tokens(cfg, 2, 32, 9)
    p = _plan(cfg, wq, dtype)
    for sel in (dw, {"wq": dw["wq"]}, {"rms_ffn_weight": dw["rms_ffn_weight"], "token_embedding_table": dw["token_embedding_table"]}):
        ref_p, ref_t = O.jvp_sequence(tokens, cfg, {k: v.double() for k, v in wq.items()}, {k: v.double() for k, v in sel.items()})
        logits, dlogits = p.forward_jvp(tokens, {k: v.to(DEV) for k, v in sel.items()})
        torch.cuda.synchronize()
        assert B.device_status() == 0
        assert _norm_rel(logits, ref_p) < (1e-4 if dtype == torch.float32 else 2e-2)
        assert _norm_rel(dlogits, ref_t) < tol, (sorted(sel), _norm_rel(dlogits, ref_t))


RAGGED = dict(dim=768, hidden_dim=2048, n_layers=2, n_heads=12, n_kv_heads=12, vocab_size=2048, seq_len=256)


def test_forward_and_vjp_bf16_on_ragged_shapes():
    """Sequence length 200 (not a multiple of the 128-row tiles of the tensor-core GEMM and attention kernels) and an odd
    batch: 600 rows leave ragged last tiles in every GEMM (M and K tails), in the attention forward and in both backward
    attention passes.  Head size 64, so the tcgen05 kernels run."""
    batch, seq = 3, 200
    p, tok, dlogits, saved, leaves = _grad_check(RAGGED, torch.bfloat16, batch, seq, 3e-2, 0.05)
    w = O.make_weights(RAGGED, 7, torch.float32, std=0.05, gains_one=False)
    wq = {k: v.bfloat16() for k, v in w.items()}
    ref = O.forward_sequence(O.make_tokens(RAGGED, batch, seq, 9), RAGGED, {k: v.float() for k, v in wq.items()})
    got = p.forward(tok)
    torch.cuda.synchronize()
    assert B.device_status() == 0
    assert _norm_rel(got, ref) < 2e-2


def test_forward_bf16_with_widths_no_tile_divides():
    """hidden 1376 and vocabulary 4000 are the per-rank widths of the 7B shape under 8-way tensor parallelism: the
    gate|up product is 2752 columns wide and the logits 4000, which no tile width of the CTA-pair GEMM divides (a partly
    filled last column of tiles, through the SwiGLU and the fp32 epilogues).  8192 tokens so that those GEMMs run."""
    cfg = dict(dim=256, hidden_dim=1376, n_layers=1, n_heads=4, n_kv_heads=4, vocab_size=4000, seq_len=1024)
    w = O.make_weights(cfg, 31, torch.float32, std=0.05)
    wb = {k: v.bfloat16() for k, v in w.items()}
    tokens = O.make_tokens(cfg, 8, 1024, 32)
    with torch.no_grad():
        ref = O.forward_sequence(tokens, cfg, {k: v.float() for k, v in wb.items()})
    p = _plan(cfg, wb, torch.bfloat16)
    got = p.forward(tokens.int().to(DEV))
    torch.cuda.synchronize()
    assert B.device_status() == 0
    assert _norm_rel(got, ref) < 2e-2
