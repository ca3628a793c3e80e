"""Greedy decode loop on the device: prefill, KV pages from an allocator, argmax sampling without a host round trip."""
import pytest
import torch

import b200_llama as B
from oracle import llama_ref as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
CFG = dict(dim=128, hidden_dim=256, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=512, seq_len=64)


def test_argmax_matches_torch_including_ties():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(37, 32000, generator=g)
    x[3, 100] = x[3, 20000] = 50.0      # equal maxima: the lower index wins
    x[5, :] = -1.0                      # a constant row: index 0
    xs = x.to(DEV)
    assert torch.equal(B.argmax(xs).cpu().long(), torch.argmax(x, dim=1))
    view = xs[:, 64:8000]               # a column window of a wider matrix (row stride != cols)
    assert torch.equal(B.argmax(view).cpu().long(), torch.argmax(x[:, 64:8000], dim=1))
    assert int(B.argmax(xs)[3]) == 100 and int(B.argmax(xs)[5]) == 0


def _oracle_greedy(cfg, w64, prompt, n_new):
    """Greedy continuation by the CPU oracle (full re-forward per token); also returns the smallest top-2 logit gap."""
    seq = prompt.clone()
    min_gap = float("inf")
    for _ in range(n_new):
        logits = O.forward_sequence(seq, cfg, w64)[:, -1, :]
        top2 = torch.topk(logits, 2, dim=1).values
        min_gap = min(min_gap, float((top2[:, 0] - top2[:, 1]).min()))
        seq = torch.cat([seq, torch.argmax(logits, dim=1, keepdim=True)], dim=1)
    return seq, min_gap


def test_generate_fp32_equals_the_oracle_greedy_loop():
    w = O.make_weights(CFG, 21, torch.float32, std=0.1, gains_one=False)
    prompt = O.make_tokens(CFG, 3, 10, 4)
    ref, gap = _oracle_greedy(CFG, {k: v.double() for k, v in w.items()}, prompt, 9)
    assert gap > 1e-3, "the seed gives a near tie; argmax equality would not be a fair bar"
    p = B.Plan(CFG, torch.float32)
    p.pack_weights({k: v.to(DEV) for k, v in w.items()})
    # a shared pool larger than needed, partly in use: the sequences get non-contiguous, out-of-order pages
    pool = p.new_kv_pages(12, 8)
    alloc = B.PageAllocator(12)
    held = alloc.alloc(5)
    alloc.free([held[1], held[3]])
    free_before = alloc.free_pages
    out = p.generate(prompt.int().to(DEV), 9, page_size=8, kv_pages=pool, allocator=alloc)
    torch.cuda.synchronize()
    assert B.device_status() == 0
    assert torch.equal(out.cpu().long(), ref)
    assert alloc.free_pages == free_before          # the sequences' pages went back to the pool
    # same tokens from a private pool with the default page size
    assert torch.equal(p.generate(prompt.int().to(DEV), 9).cpu().long(), ref)


def test_generate_bf16_runs_and_rejects_bad_requests():
    w = O.make_weights(CFG, 22, torch.float32, std=0.1)
    p = B.Plan(CFG, torch.bfloat16)
    p.pack_weights({k: v.bfloat16().to(DEV) for k, v in w.items()})
    prompt = O.make_tokens(CFG, 2, 12, 5).int().to(DEV)
    out = p.generate(prompt, 6, page_size=16)
    assert out.shape == (2, 18) and torch.equal(out[:, :12], prompt)
    assert int(out.min()) >= 0 and int(out.max()) < CFG["vocab_size"]
    with pytest.raises(B.B200Error):
        p.generate(prompt, 60)                      # 72 positions > seq_len 64
    with pytest.raises(B.B200Error):
        p.generate(prompt, 6, page_size=16, kv_pages=p.new_kv_pages(1, 16), allocator=B.PageAllocator(1))  # pool too small
    assert B.device_status() == 0
