"""Worker for the multi-GPU parity tests; launched with torch.distributed.run, one rank per GPU.

Checks, against the CPU oracle: tensor-parallel forward (vocabulary-sharded logits), tensor-parallel decode steps,
and the data-parallel gradient all-reduce."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "enzyme-jax_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch
import torch.distributed as dist

import b200_llama as B
from oracle import llama_ref as O


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = B.Comm(rank, world, symmetric=os.environ.get("B200_TEST_SYMM", "1") == "1")
    if rank == 0:
        print("PEER_MEMORY", comm.peer_memory())
    cfg = dict(dim=256, hidden_dim=512, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=1024, seq_len=160)
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 2e-2)):
        w = {k: v.to(dtype) for k, v in O.make_weights(cfg, 3, torch.float32, std=0.05).items()}
        tokens = O.make_tokens(cfg, 2, 128, 4)
        ref = O.forward_sequence(tokens, cfg, {k: v.double() for k, v in w.items()})
        plan = B.Plan(cfg, dtype, tp_rank=rank, tp_size=world, comm=comm)
        plan.pack_weights({k: v.cuda().contiguous() for k, v in w.items()})
        got = plan.forward(tokens.int().cuda())
        torch.cuda.synchronize()
        vl = cfg["vocab_size"] // world
        mine = ref[..., rank * vl:(rank + 1) * vl]
        err = float((got.double().cpu() - mine).abs().max() / ref.abs().max())
        assert err < tol, ("tp forward", dtype, err)
        # decode, tensor parallel: the cache holds this rank's heads only
        page, seq = 32, 40
        max_pages = (seq + page - 1) // page
        kv = plan.new_kv_pages(2 * max_pages, page)
        table = torch.arange(2 * max_pages, dtype=torch.int32, device="cuda").view(2, max_pages)
        tok = tokens.int().cuda()
        for pos in range(seq):
            _, lg = plan.decode_step(pos, kv, table, tokens=tok[:, pos].contiguous())
            e = float((lg.double().cpu() - mine[:, pos]).abs().max() / ref.abs().max())
            assert e < tol, ("tp decode", dtype, pos, e)
        assert B.device_status() == 0
        if dtype == torch.bfloat16:
            # a tensor-parallel plan refuses graph capture (the peer exchange numbers its rounds from the host)
            try:
                plan.capture_forward(tokens.int().cuda(), got)
                raise AssertionError("capture of a tensor-parallel plan must be refused")
            except B.B200Error as e:
                assert e.status == 10
        plan.close()
    # an odd batch (cannot be split into two halves), and an even batch with the two-half pipeline forced on
    for env_off, nb in ((None, 3), ("B200_TP_PIPELINE", 2)):
        if env_off:
            os.environ[env_off] = "1"   # the two-half pipeline is off by default: force it here
        w = {k: v.bfloat16() for k, v in O.make_weights(cfg, 3, torch.float32, std=0.05).items()}
        tokens = O.make_tokens(cfg, nb, 128, 4)
        ref = O.forward_sequence(tokens, cfg, {k: v.double() for k, v in w.items()})
        plan = B.Plan(cfg, torch.bfloat16, tp_rank=rank, tp_size=world, comm=comm)
        plan.pack_weights({k: v.cuda().contiguous() for k, v in w.items()})
        got = plan.forward(tokens.int().cuda())
        torch.cuda.synchronize()
        vl = cfg["vocab_size"] // world
        err = float((got.double().cpu() - ref[..., rank * vl:(rank + 1) * vl]).abs().max() / ref.abs().max())
        assert err < 2e-2, ("tp forward, pipeline forced on" if env_off else "tp forward, odd batch", err)
        plan.close()
        if env_off:
            del os.environ[env_off]
    # the same forward through the all-reduce per block (row sharding off): the path taken when peer memory is absent
    os.environ["B200_TP_ROW_SHARD"] = "0"
    w = {k: v.bfloat16() for k, v in O.make_weights(cfg, 3, torch.float32, std=0.05).items()}
    tokens = O.make_tokens(cfg, 2, 128, 4)
    ref = O.forward_sequence(tokens, cfg, {k: v.double() for k, v in w.items()})
    plan = B.Plan(cfg, torch.bfloat16, tp_rank=rank, tp_size=world, comm=comm)
    plan.pack_weights({k: v.cuda().contiguous() for k, v in w.items()})
    got = plan.forward(tokens.int().cuda())
    torch.cuda.synchronize()
    vl = cfg["vocab_size"] // world
    err = float((got.double().cpu() - ref[..., rank * vl:(rank + 1) * vl]).abs().max() / ref.abs().max())
    assert err < 2e-2, ("tp forward, all-reduce path", err)
    plan.close()
    del os.environ["B200_TP_ROW_SHARD"]
    # 2 x 1024 tokens, with the two-half pipeline on
    os.environ["B200_TP_PIPELINE"] = "1"
    cfg_long = dict(cfg, seq_len=1024)
    w = {k: v.bfloat16() for k, v in O.make_weights(cfg_long, 8, torch.float32, std=0.05).items()}
    tokens = O.make_tokens(cfg_long, 2, 1024, 9)
    ref = O.forward_sequence(tokens, cfg_long, {k: v.float() for k, v in w.items()})
    plan = B.Plan(cfg_long, torch.bfloat16, tp_rank=rank, tp_size=world, comm=comm)
    plan.pack_weights({k: v.cuda().contiguous() for k, v in w.items()})
    for _ in range(3):  # repeated calls reuse the fork/join events
        got = plan.forward(tokens.int().cuda())
    torch.cuda.synchronize()
    vl = cfg_long["vocab_size"] // world
    err = float((got.cpu() - ref[..., rank * vl:(rank + 1) * vl]).abs().max() / ref.abs().max())
    assert err < 2e-2, ("tp forward, long", err)
    # rows 7 of 8 per rank are a ragged share: T = 2 * 1000 tokens over the ranks
    tok_r = tokens[:, :1000].contiguous()
    ref_r = O.forward_sequence(tok_r, cfg_long, {k: v.float() for k, v in w.items()})
    got_r = plan.forward(tok_r.int().cuda())
    torch.cuda.synchronize()
    err = float((got_r.cpu() - ref_r[..., rank * vl:(rank + 1) * vl]).abs().max() / ref_r.abs().max())
    assert err < 2e-2, ("tp forward, 2000 tokens", err)
    # the warm-up tuner times both exchange schedules; all ranks keep the same one; either gives the same logits
    tok_dev = tokens.int().cuda()
    res = plan.tune_tensor_parallel(tok_dev)
    assert res["tp_pipeline"] in (0, 1) and plan.get_option("tp_pipeline") == res["tp_pipeline"], res
    assert res["one_batch_ms"] > 0 and res["two_halves_ms"] > 0, res
    agreed = torch.tensor([res["tp_pipeline"], -res["tp_pipeline"]], device="cuda")
    dist.all_reduce(agreed, op=dist.ReduceOp.MAX)
    assert int(agreed[0]) == -int(agreed[1]), "ranks disagree on the exchange schedule"
    for mode in (0, 1):
        plan.set_option("tp_pipeline", mode)
        got_m = plan.forward(tok_dev)
        torch.cuda.synchronize()
        err = float((got_m.cpu() - ref[..., rank * vl:(rank + 1) * vl]).abs().max() / ref.abs().max())
        assert err < 2e-2, ("tp forward after tuning", mode, err)
        assert float((got_m - got).abs().max()) <= 1e-3 * float(ref.abs().max()), ("schedules differ", mode)
    try:
        plan.set_option("no_such_option", 1)
        raise AssertionError("an unknown option must be refused")
    except B.B200Error as e:
        assert e.status == 1
    assert B.device_status() == 0
    plan.close()
    del os.environ["B200_TP_PIPELINE"]
    # the widths of the 7B shape (2 layers, 2 x 1024 tokens): here the row-parallel projections run on the CTA-pair
    # GEMM, which stores every band of rows of the partial product straight into its owner's memory (pushed store);
    # the same forward with the pull form must give the same logits, and both the oracle's
    cfg7 = dict(dim=4096, hidden_dim=11008, n_layers=2, n_heads=32, n_kv_heads=32, vocab_size=32768, seq_len=1024)
    w = {k: v.bfloat16() for k, v in O.make_weights(cfg7, 21, torch.float32, std=0.02).items()}
    tokens = O.make_tokens(cfg7, 2, 1024, 22)
    ref = O.forward_sequence(tokens, cfg7, {k: v.float() for k, v in w.items()})
    plan = B.Plan(cfg7, torch.bfloat16, tp_rank=rank, tp_size=world, comm=comm)
    plan.pack_weights({k: v.cuda().contiguous() for k, v in w.items()})
    del w
    vl = cfg7["vocab_size"] // world
    tok_dev = tokens.int().cuda()
    # ... and the column-parallel projections wait for the gathered rows band by band (the exchange kernel returns
    # once this rank's rows are delivered); every combination of the two must give the same logits
    outs = {}
    for push, bands in ((1, 1), (0, 1), (1, 0), (0, 0)):
        plan.set_option("tp_push", push)
        plan.set_option("tp_bands", bands)
        for _ in range(3):  # repeatedly: slots, gathered rows and flag words are reused by the next exchange
            got = plan.forward(tok_dev)
        torch.cuda.synchronize()
        assert plan.get_option("tp_push_last") == push, ("pushed store taken?", push, plan.get_option("tp_push_last"))
        assert plan.get_option("tp_bands_last") == bands, ("banded consumers taken?", bands)
        err = float((got.cpu() - ref[..., rank * vl:(rank + 1) * vl]).abs().max() / ref.abs().max())
        assert err < 2e-2, ("tp forward at the 7B widths", push, bands, err)
        outs[(push, bands)] = got.clone()
        assert B.device_status() == 0, (push, bands)
    for k, v in outs.items():
        assert torch.equal(v, outs[(0, 0)]), ("pushed / banded forms must give the same logits as the plain form", k)
    assert B.device_status() == 0
    plan.close()
    # data parallel: each rank differentiates its own sequences, gradients are summed over the ranks
    dtype = torch.float32
    w = O.make_weights(cfg, 5, torch.float32, std=0.05, gains_one=False)
    tokens = O.make_tokens(cfg, 2 * world, 64, 6)
    g = torch.Generator().manual_seed(7)
    dl = torch.randn(2 * world, 64, cfg["vocab_size"], generator=g)
    _, ref = O.vjp_sequence(tokens, cfg, {k: v.double() for k, v in w.items()}, dl.double())
    plan = B.Plan(cfg, dtype)
    plan.pack_weights({k: v.cuda().contiguous() for k, v in w.items()}, with_transposed=True)
    tok = tokens[2 * rank:2 * rank + 2].int().cuda().contiguous()
    saved = plan.new_saved(2, 64)
    plan.forward(tok, saved=saved)
    grads = plan.backward(tok, dl[2 * rank:2 * rank + 2].cuda().contiguous(), saved, plan.new_grads())
    comm.allreduce_f32(grads)
    leaves = plan.unpack_grads(grads)
    for k, r in ref.items():
        e = float((leaves[k].double().cpu() - r).abs().max() / r.abs().max())
        assert e < 1e-4, ("dp grads", k, e)
    torch.cuda.synchronize()
    dist.barrier()
    comm.destroy()
    dist.destroy_process_group()
    if rank == 0:
        print("MULTI_GPU_OK", world)


if __name__ == "__main__":
    main()
