"""Benchmark of the llama forward / VJP hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c2|c1|c3|c5] [--impl reference]

Default: the Llama-2-7B-shape bf16 prefill forward (dim 4096, 32 layers, batch 4 x
2048 tokens), the largest single-GPU configuration, tensor parallel over all N
ranks (N = 1: one GPU holds the whole model); one step = one forward over the
batch, tokens/s of the whole job.  For N > 1 launch under
``torch.distributed.run`` (one rank per GPU, NCCL + peer memory over NVLink).
Prints ONE JSON line on rank 0's standard output; everything else any rank or
library prints (NCCL's log included) goes to standard error.

``--impl reference`` times the CPU restatement of the reference model (the
oracle, torch-CPU fp32 on all host threads) on a bounded sample of the same
workload: the reference itself (JAX/XLA) is not installable here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "enzyme-jax_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch

C2 = dict(dim=768, hidden_dim=2048, n_layers=12, n_heads=12, n_kv_heads=12, vocab_size=32000, seq_len=1024)
C1 = dict(dim=288, hidden_dim=768, n_layers=6, n_heads=6, n_kv_heads=6, vocab_size=32000, seq_len=256)
C4 = dict(dim=4096, hidden_dim=11008, n_layers=32, n_heads=32, n_kv_heads=32, vocab_size=32000, seq_len=2048)

L2_BYTES = 126 * 1024 * 1024

WORKLOADS = {
    # name: (config, dtype, batch per step, seq, description)
    "c2": (C2, "bf16", 8, 1024, "llama-110M prefill forward, batch 8 x 1024 tokens, bf16 weights/activations, fp32 accumulate"),
    "c1": (C1, "f32", 1, 256, "llama2.c 15M forward, batch 1 x 256 tokens, fp32"),
    "c3": (C2, "bf16", 64, 1024, "llama-110M forward + VJP wrt all weights, global batch 64 x 1024, data parallel"),
    "c4": (C4, "bf16", 4, 2048, "llama-2-7B shape prefill forward, batch 4 x 2048, tensor parallel"),
    "c5": (C4, "bf16", 64, 4096, "llama-2-7B shape decode, batch 64, 4096-token KV cache, 128 steps, tensor parallel"),
}


def fwd_flops(cfg, batch, seq):
    L, d, h, V = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
    W = L * (4 * d * d + 3 * d * h) + V * d
    T = batch * seq
    return 2.0 * T * W + 4.0 * seq * seq * d * L * batch / 2.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops_burst=p["bf16_tflops"], tflops_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


KERNEL_OF_CLASS = {
    "gemm_tcgen05_pair": "gemm_tc2_kernel", "gemm_tcgen05": "gemm_tc_kernel", "gemm_ffma": "gemm_simt_kernel",
    "attention_fwd": "attn_fwd_tc_kernel", "attention_bwd": "attn_bwd_tc_kernel",
    "attention_decode": "attn_decode_vec_kernel", "allreduce": "peer_rownorm_kernel",
}


def _profile_table_rows(name):
    """Rows of the markdown table in profiles/<name> as lists of cell strings (no header, no rule)."""
    path = os.path.join(ROOT, "profiles", name)
    if not os.path.exists(path):
        return []
    rows = []
    for ln in open(path):
        cells = [c.strip() for c in ln.strip().strip("|").split("|")]
        if ln.lstrip().startswith("|") and len(cells) >= 3 and not set(cells[0]) <= set("-: "):
            rows.append(cells)
    return rows


def traffic_from_profiles(workload, kernel):
    """DRAM bytes per launch of `kernel` in `workload`, read from the table of ncu captures kept in
    profiles/dram_traffic_per_launch.md (columns: workload, kernel, bytes per launch, capture).  None when no
    capture of that pair has been recorded: the number is never a constant of this file."""
    for cells in _profile_table_rows("dram_traffic_per_launch.md"):
        if cells[0] == workload and cells[1] == kernel:
            try:
                return float(cells[2]), "profiles/dram_traffic_per_launch.md: " + (cells[3] if len(cells) > 3 else "")
            except ValueError:
                pass
    return None, None


def fp32_peak_from_profiles():
    """Measured FFMA rate of the GPU in TFLOP/s (profiles/fp32_ffma_peak.md, a table row `fp32_ffma | <TFLOP/s> | how`)."""
    for cells in _profile_table_rows("fp32_ffma_peak.md"):
        if cells[0] == "fp32_ffma":
            try:
                return float(cells[1])
            except ValueError:
                pass
    return None


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU during the timed region: NVML in a background thread
    (read-only queries), or an `nvidia-smi -lms` child process when the NVML binding is missing."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, gpu_index: int, period_s: float = 0.1):
        self.gpu = gpu_index
        self.period = float(os.environ.get("B200_CLOCK_PERIOD_S", period_s))
        self.lines = []
        self.samples = []
        self.proc = None
        self.thread = None
        self.stop_flag = threading.Event()
        self.max_mhz = None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if self.gpu < len(ids) and ids[self.gpu].isdigit():
                return int(ids[self.gpu])
        return self.gpu

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self._physical_index()), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.reader = threading.Thread(target=self._read, daemon=True)
            self.reader.start()
        except Exception:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((mhz, mask))
            except Exception:
                pass
            self.stop_flag.wait(self.period)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            sm = sorted(x[0] for x in self.samples)
            reasons = set()
            for _, mask in self.samples:
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        reasons.add(name)
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(reasons), "samples": len(sm), "source": "nvml"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1]))
                mx = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


def cpu_oracle_rate(cfg, seq, sample_batch, reps, vjp=False):
    """tokens/s of the oracle (torch-CPU fp32, all host threads) on a bounded sample."""
    from oracle import llama_ref as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    w = O.make_weights(cfg, 2, torch.float32)
    tokens = O.make_tokens(cfg, sample_batch, seq, 2)
    dl = torch.randn(sample_batch, seq, cfg["vocab_size"]) if vjp else None

    def step():
        if vjp:
            O.vjp_sequence(tokens, cfg, w, dl)
        else:
            with torch.no_grad():
                O.forward_sequence(tokens, cfg, w)

    step()
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        step()
        best = min(best, time.perf_counter() - t0)
    return sample_batch * seq / best, threads, best


def cpu_extrapolated_7b(cfg, batch, seq, reps, past=0):
    """Seconds per step (`batch` sequences of `seq` new tokens, `past` cached rows each) of the full-depth 7B-shape
    oracle, from timing a 1-layer and a 2-layer model of the same widths (embedding, final norm and the logits
    projection are in both): t(L) = t1 + (L - 1) * (t2 - t1)."""
    from oracle import llama_ref as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    best = {}
    w2 = O.make_weights(dict(cfg, n_layers=2), 2, torch.float32)
    tokens = O.make_tokens(cfg, batch, seq, 2)
    pk = pv = None
    if past:
        g = torch.Generator().manual_seed(3)
        pk = torch.randn(2, batch, past, cfg["dim"], generator=g)
        pv = torch.randn(2, batch, past, cfg["dim"], generator=g)
    for layers in (1, 2):
        c = dict(cfg, n_layers=layers)
        w = {k: (v[:layers] if v.dim() == 3 or k in ("rms_att_weight", "rms_ffn_weight") else v) for k, v in w2.items()}
        b = float("inf")
        for _ in range(reps + 1):  # the first pass warms the thread pool and the allocator
            t0 = time.perf_counter()
            with torch.no_grad():
                O.forward_sequence(tokens, c, w, past_k=pk[:layers] if past else None,
                                   past_v=pv[:layers] if past else None)
            b = min(b, time.perf_counter() - t0)
        best[layers] = b
    per_layer = max(best[2] - best[1], 1e-9)
    return best[1] + (cfg["n_layers"] - 1) * per_layer, threads, best


def run_reference(args, rank, world):
    if rank != 0:
        return None
    cfg, dtype, batch, seq, desc = WORKLOADS[args.workload]
    from oracle import llama_ref as O  # noqa: F401
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    steps = max(1, min(args.steps, 5))
    if args.workload in ("c4", "c5"):
        prefill = args.workload == "c4"
        sb, ss, past = (1, seq, 0) if prefill else (8, 1, seq)  # decode: 8 sequences, one new token, 4096 cached rows
        secs = []
        for _ in range(min(steps, 2)):
            t_full, threads, best = cpu_extrapolated_7b(cfg, sb, ss, 1, past)
            secs.append(t_full)
        dt = min(secs)
        value = sb * ss / dt
        what = f"1 sequence of {ss} tokens" if prefill else f"{sb} sequences, one new token each over {past} cached rows"
        sample = (f"EXTRAPOLATED: {what} through a 1-layer and a 2-layer model of the 7B widths "
                  f"(torch-CPU fp32 oracle, {best[1]:.2f} s and {best[2]:.2f} s per step); full depth = t1 + 31 * (t2 - t1); "
                  "embedding, final norm and the 32000-wide logits projection are in t1")
        steps = len(secs)
    else:
        w = O.make_weights(cfg, 2, torch.float32)
        tokens = O.make_tokens(cfg, 1, seq, 2)
        vjp = args.workload == "c3"
        dl = torch.randn(1, seq, cfg["vocab_size"]) if vjp else None

        def step():
            if vjp:
                O.vjp_sequence(tokens, cfg, w, dl)
            else:
                with torch.no_grad():
                    O.forward_sequence(tokens, cfg, w)

        for _ in range(max(1, min(args.warmup, 1))):
            step()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        dt = (time.perf_counter() - t0) / steps
        value = tokens.shape[1] / dt
        sample = f"1 sequence of {tokens.shape[1]} tokens per step, {steps} steps, torch-CPU fp32 oracle"
    return {
        "impl": "reference", "metric": "tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.workload in ("c3", "c4", "c5") else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOADS[args.workload][4]},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference (JAX/XLA) is not installable here; this is the CPU restatement of test/llama.py",
    }


def synth_weights(cfg, dtype, device, seed=1):
    """Random-init weights of the architecture, generated on the device from a seed."""
    L, d, h, V = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
    shapes = {
        "rms_att_weight": (L, d), "rms_ffn_weight": (L, d), "rms_final_weight": (d,),
        "token_embedding_table": (V, d), "w1": (L, h, d), "w2": (L, d, h), "w3": (L, h, d), "wcls": (V, d),
        "wk": (L, d, d), "wo": (L, d, d), "wq": (L, d, d), "wv": (L, d, d),
    }
    g = torch.Generator(device=device).manual_seed(seed)
    w = {}
    for name in sorted(shapes):
        if name.startswith("rms_"):
            w[name] = torch.ones(shapes[name], dtype=dtype, device=device)
        else:
            w[name] = torch.empty(shapes[name], dtype=dtype, device=device).normal_(0.0, 0.02, generator=g)
    return w


def timed(fn, steps, world, dist, flush=None):
    """K steps bracketed by barrier + synchronize, CUDA events on the current stream, max over ranks.
    With `flush` (a callable that overwrites a buffer larger than L2) every step gets its own event pair and the
    flush runs between the pairs, outside the time that is summed."""
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    if flush is None:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        total = a.elapsed_time(b)
    else:
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for i, (a, b) in enumerate(pairs):
            flush()
            a.record()
            fn(i)
            b.record()
        torch.cuda.synchronize()
        total = sum(a.elapsed_time(b) for a, b in pairs)
    ms = torch.tensor([total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.barrier()
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def run_prefill(args, rank, world, local, B, dist):
    cfg, dname, batch, seq, desc = WORKLOADS[args.workload]
    if args.batch > 0:
        batch = args.batch
        desc += f" [batch overridden to {batch}]"
    if args.layers > 0:
        cfg = dict(cfg, n_layers=args.layers)
        desc += f" [layers overridden to {args.layers}]"
    dtype = torch.bfloat16 if dname == "bf16" else torch.float32
    dev = torch.device("cuda", local)
    pk = peaks()
    tp = world if args.workload == "c4" else 1
    comm = B.Comm(rank, world) if tp > 1 else None
    plan = B.Plan(cfg, dtype, tp_rank=rank if tp > 1 else 0, tp_size=tp, comm=comm)
    w = synth_weights(cfg, dtype, dev)
    plan.pack_weights(w)
    del w
    torch.cuda.empty_cache()

    gen = torch.Generator().manual_seed(100 + (0 if tp > 1 else rank))
    n_bufs = 4
    host_tokens = [torch.randint(0, cfg["vocab_size"], (batch, seq), generator=gen, dtype=torch.int32).pin_memory()
                   for _ in range(n_bufs)]
    dev_tokens = [t.to(dev) for t in host_tokens]
    logits = torch.empty(batch, seq, plan.vocab_local, dtype=torch.float32, device=dev)
    tok_stage = torch.empty(batch, seq, dtype=torch.int32, device=dev)

    # The plan's kernel sequence is static: replay it as a CUDA graph (one graph per token buffer).
    use_graph = not args.no_graph and tp == 1
    launches_per_forward = None
    if use_graph:
        l_before = B.launch_count()
        graphs = [plan.capture_forward(t, logits) for t in dev_tokens]
        launches_per_forward = (B.launch_count() - l_before) // (2 * n_bufs)
    last_dev = torch.empty(batch, plan.vocab_local, dtype=torch.float32, device=dev)

    # Tensor parallel: --tune-tp times the two exchange schedules (one batch / two halves in flight) before the
    # warm-up and keeps the faster one on every rank; without it the plan's default (one batch) runs.
    tuned = None
    if args.tune_tp and tp > 1 and comm.peer_memory() and os.environ.get("B200_TP_ROW_SHARD", "1") != "0":
        tuned = plan.tune_tensor_parallel(dev_tokens[0], logits)

    def step_resident(i):
        if use_graph:
            graphs[i % n_bufs].replay()
        else:
            plan.forward(dev_tokens[i % n_bufs], logits=logits)

    # End to end: every step uploads its tokens from pinned host memory, runs the forward and brings the
    # last-position logits back to pinned host memory.  The loop is the double-buffered one a server
    # runs: the host enqueues step i while step i-1 computes, and consumes the result of step i-2
    # (waits for its copy, reads it) before it reuses that host buffer.
    depth = 2
    last_hosts = [torch.empty(batch, plan.vocab_local, dtype=torch.float32).pin_memory() for _ in range(depth)]
    done = [torch.cuda.Event() for _ in range(depth)]
    pending = [False] * depth
    consumed = []

    if use_graph:  # n_bufs is a multiple of depth: host buffer j always pairs with result slot j % depth
        graphs_e2e = [plan.capture_prefill_step(host_tokens[j], tok_stage, logits, last_dev, last_hosts[j % depth])
                      for j in range(n_bufs)]

    def consume(slot):
        done[slot].synchronize()
        consumed.append(float(last_hosts[slot][0, 0]))  # the host reads the result
        pending[slot] = False

    def step_e2e(i):
        slot = i % depth
        if pending[slot]:
            consume(slot)
        if use_graph:
            graphs_e2e[i % n_bufs].replay()  # upload, forward, gather and download are nodes of one graph
        else:
            tok_stage.copy_(host_tokens[i % n_bufs], non_blocking=True)
            plan.forward(tok_stage, logits=logits)
            last_dev.copy_(logits[:, -1, :])
            last_hosts[slot].copy_(last_dev, non_blocking=True)
        done[slot].record()
        pending[slot] = True
        if i == args.steps - 1:  # drain inside the timed region
            for k in range(1, depth + 1):
                if pending[(slot + k) % depth]:
                    consume((slot + k) % depth)

    for i in range(args.warmup):
        step_resident(i)
    for i in range(args.warmup):  # the end-to-end path has its own graph and copy kernels: warm them too
        if use_graph:
            graphs_e2e[i % n_bufs].replay()
        else:
            tok_stage.copy_(host_tokens[i % n_bufs], non_blocking=True)
            plan.forward(tok_stage, logits=logits)
            last_dev.copy_(logits[:, -1, :])
            last_hosts[i % depth].copy_(last_dev, non_blocking=True)
    torch.cuda.synchronize()
    if B.device_status() != 0:
        raise RuntimeError("device status word set during warm-up")

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # A working set (weights + logits) that L2 could hold from one step to the next is evicted between steps.
    working_set = plan.packed.numel() + logits.numel() * 4
    flush = None
    if working_set < 2 * L2_BYTES:
        flush_buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)
        flush = flush_buf.zero_
    l0 = B.launch_count()
    ms = timed(step_resident, args.steps, world, dist, flush)
    launches = (B.launch_count() - l0) if not use_graph else launches_per_forward * args.steps
    ms_e2e = timed(step_e2e, args.steps, world, dist, flush)
    clocks = sampler.stop() if rank == 0 else None

    # per-kernel event timing over the same K steps (a second pass, eager launches: the event
    # pairs cost a little, so they are kept out of the headline timing)
    B.profile_enable(True)
    timed(lambda i: plan.forward(dev_tokens[i % n_bufs], logits=logits), args.steps, world, dist)
    prof = B.profile_read()
    B.profile_enable(False)
    if B.device_status() != 0:
        raise RuntimeError("device status word set during the timed region")

    replicas = 1 if tp > 1 else world
    tokens_per_step = batch * seq * replicas
    value = tokens_per_step / (ms / args.steps / 1e3)
    e2e = tokens_per_step / (ms_e2e / args.steps / 1e3)
    dom_name = max(("gemm_tcgen05_pair", "gemm_tcgen05", "gemm_ffma", "attention_fwd"), key=lambda k: prof[k]["ms"])
    dom = prof[dom_name]
    tensor_bound = dname == "bf16"
    ach = dom["work"] / (dom["ms"] / 1e3) / 1e12 if dom["ms"] > 0 else 0.0
    peak, peak_burst = pk["tflops_sustained"], pk["tflops_burst"]
    full_size = args.batch == 0 and args.layers == 0
    traffic, traffic_src = traffic_from_profiles(args.workload, KERNEL_OF_CLASS[dom_name]) if full_size else (None, None)
    step_flops = fwd_flops(cfg, batch, seq) / tp
    roofline = {
        "bound": "tensor", "kernel": KERNEL_OF_CLASS[dom_name], "achieved": ach, "peak": peak, "unit": "TFLOP/s",
        "frac": ach / peak, "peak_burst": peak_burst, "frac_burst": ach / peak_burst,
        "traffic": traffic, "traffic_unit": "DRAM bytes per launch, mean over this kernel's launches of one step (ncu)",
        "traffic_source": traffic_src,
        "peak_source": pk["source"] + " (bf16 matmul: `peak` is the seconds-long figure under the power cap, "
                                      "`peak_burst` the best of 10 isolated runs)",
        "launches": dom["launches"], "kernel_ms_per_step": dom["ms"] / args.steps,
        "share_of_step": dom["ms"] / max(1e-9, sum(v["ms"] for v in prof.values())),
        "whole_step_frac": step_flops / (ms / args.steps / 1e3) / 1e12 / peak,
        "whole_step_frac_burst": step_flops / (ms / args.steps / 1e3) / 1e12 / peak_burst,
        "kernels_ms_per_step": {k: v["ms"] / args.steps for k, v in prof.items() if v["launches"]},
    }
    if not tensor_bound:
        fp32 = fp32_peak_from_profiles()
        roofline["note"] = ("fp32 configuration: FFMA kernels; `frac` is against the bf16 tensor peak for reference only, "
                            "`frac_fp32` against the measured FFMA rate of the GPU")
        roofline["peak_fp32"] = fp32
        roofline["frac_fp32"] = ach / fp32 if fp32 else None
    line = {
        "metric": "tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": dname, "data": "synthetic",
        "config": {"workload": desc, "batch_per_rank": batch, "seq_len": seq,
                   "parallelism": f"tp{tp}" if tp > 1 else (f"replicas{world}" if world > 1 else "single"),
                   "l2_policy": (f"working set per step (weights + logits, {working_set / 1e6:.0f} MB) exceeds the 126 MB "
                                 "L2; token buffers rotate" if flush is None else
                                 f"working set per step ({working_set / 1e6:.0f} MB) would fit the 126 MB L2: a 252 MB "
                                 "buffer is overwritten between steps, outside the per-step event pairs that are summed"),
                   "launch": "cuda graph replay" if use_graph else "eager launches"},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": batch * seq * 4,
                "d2h_bytes_per_step": batch * plan.vocab_local * 4, "ms_per_step": ms_e2e / args.steps,
                "result": "last-position logits of every sequence",
                "pipeline": "double-buffered host loop: step i is enqueued while step i-1 computes; the host waits "
                            "for and reads the result of step i-2 before reusing its buffer; drained inside the "
                            "timed region"},
        "gpu_launches": launches, "roofline": roofline, "clocks": clocks,
    }
    if tp > 1:
        mode = comm.peer_memory()
        fused = mode and os.environ.get("B200_TP_ROW_SHARD", "1") != "0"
        line["config"]["exchange"] = (
            ("row-sharded residual stream: one fused reduce + add + RMSNorm + gather kernel per block, "
             + ("summed inside the NVLink switch (multimem.ld_reduce / multimem.st)"
                if mode == 2 and (os.environ.get("B200_TP_MULTIMEM", "0") != "0")
                else "plain peer loads and stores"))
            if fused else "all-reduce per block")
        if fused and plan.get_option("tp_pipeline") and batch % 2 == 0:
            line["config"]["exchange"] += ("; two halves of the batch in flight: the exchange of one half runs on a "
                                           "second stream beside the other half's GEMMs and attention")
        elif fused:
            line["config"]["exchange"] += "; one batch, the exchange between the kernels"
        if fused and plan.get_option("tp_push_last"):
            line["config"]["exchange"] += ("; the Wo / W2 GEMMs store each band of rows of their partial product "
                                           "straight into its owner's memory, tile by tile")
        if fused and plan.get_option("tp_bands_last"):
            line["config"]["exchange"] += ("; the QKV / W1|W3 / logits GEMMs wait for the gathered rows band by band, "
                                           "starting on this rank's own")
        if tuned:
            line["config"]["exchange"] += (f" (chosen by timing both before the warm-up: one batch "
                                           f"{tuned['one_batch_ms']:.2f} ms, two halves {tuned['two_halves_ms']:.2f} ms)")
        line["exchange_ms_per_step"] = prof["allreduce"]["ms"] / args.steps
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample_b = 1
        reps = 2 if args.workload != "c1" else 5
        if args.workload == "c4":
            t_full, threads, best = cpu_extrapolated_7b(cfg, 1, seq, 1)
            line["cpu_baseline"] = {
                "value": seq / t_full, "unit": "tokens/s", "cores": threads, "kind": "port",
                "sample": f"EXTRAPOLATED: 1 sequence of {seq} tokens through a 1-layer and a 2-layer model of the 7B "
                          f"widths (torch-CPU fp32 restatement of test/llama.py, {best[1]:.2f} s and {best[2]:.2f} s); "
                          f"full depth = t1 + {cfg['n_layers'] - 1} * (t2 - t1)"}
        else:
            rate, threads, best = cpu_oracle_rate(cfg, seq, sample_b, reps)
            line["cpu_baseline"] = {
                "value": rate, "unit": "tokens/s", "cores": threads, "kind": "port",
                "sample": f"{sample_b} sequence of {seq} tokens, best of {reps}, torch-CPU fp32 restatement of "
                          "test/llama.py"}
    if comm:
        comm.destroy()
    return line


def vjp_flops(cfg, batch, seq):
    """Model flops of forward + VJP: 3x the GEMM flops, 3.5x the causal-attention flops."""
    L, d, h, V = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
    W = L * (4 * d * d + 3 * d * h) + V * d
    T = batch * seq
    return 3 * 2.0 * T * W + 3.5 * 4.0 * seq * seq * d * L * batch / 2.0


def run_vjp(args, rank, world, local, B, dist):
    """Config 3: forward + reverse mode w.r.t. all weights, global batch 64 x 1024 split over the
    ranks (data parallel), 8-sequence micro-batches, one fp32 gradient all-reduce per step."""
    cfg, dname, gbatch, seq, desc = WORKLOADS["c3"]
    if args.batch > 0:
        gbatch = args.batch * world
        desc += f" [global batch overridden to {gbatch}]"
    dev = torch.device("cuda", local)
    pk = peaks()
    per_rank = gbatch // world
    micro = min(8, per_rank)
    n_micro = per_rank // micro
    comm = B.Comm(rank, world) if world > 1 else None
    plan = B.Plan(cfg, torch.bfloat16)
    w = synth_weights(cfg, torch.bfloat16, dev)
    plan.pack_weights(w, with_transposed=True)
    del w
    gen = torch.Generator().manual_seed(200 + rank)
    host_tokens = [torch.randint(0, cfg["vocab_size"], (micro, seq), generator=gen, dtype=torch.int32).pin_memory()
                   for _ in range(n_micro)]
    dev_tokens = [t.to(dev) for t in host_tokens]
    tok_stage = torch.empty(micro, seq, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(300 + rank)
    dlogits = torch.empty(micro, seq, cfg["vocab_size"], dtype=torch.float32, device=dev)
    dlogits.normal_(0.0, 1.0, generator=g)
    logits = torch.empty(micro, seq, cfg["vocab_size"], dtype=torch.float32, device=dev)
    saved = plan.new_saved(micro, seq)
    grads = plan.new_grads()
    norm_host = torch.empty(1, dtype=torch.float32).pin_memory()

    def step(i, e2e=False):
        for mb in range(n_micro):
            if e2e:
                tok_stage.copy_(host_tokens[mb], non_blocking=True)
                tok = tok_stage
            else:
                tok = dev_tokens[mb]
            plan.forward(tok, saved=saved, logits=logits)
            plan.backward(tok, dlogits, saved, grads, accumulate=mb > 0)
        if comm:
            comm.allreduce_f32(grads)
        if e2e:
            norm_host.copy_(grads[:1], non_blocking=True)
            torch.cuda.current_stream().synchronize()

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if B.device_status() != 0:
        raise RuntimeError("device status word set during warm-up")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    l0 = B.launch_count()
    ms = timed(lambda i: step(i), args.steps, world, dist)
    launches = B.launch_count() - l0
    ms_e2e = timed(lambda i: step(i, True), args.steps, world, dist)
    clocks = sampler.stop() if rank == 0 else None
    B.profile_enable(True)
    timed(lambda i: step(i), max(1, args.steps // 2), world, dist)
    prof = B.profile_read()
    B.profile_enable(False)
    psteps = max(1, args.steps // 2)
    tokens = gbatch * seq
    value = tokens / (ms / args.steps / 1e3)
    dom_name = max(prof, key=lambda k: prof[k]["ms"])
    dom = prof[dom_name]
    ach = dom["work"] / (dom["ms"] / 1e3) / 1e12 if dom["ms"] > 0 else 0.0
    peak = pk["tflops_sustained"]
    line = {
        "metric": "tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "global_batch": gbatch, "seq_len": seq, "micro_batch": micro,
                   "parallelism": f"dp{world}", "l2_policy": "per-micro-batch working set (2 GB of logits and cotangent, "
                   "1.8 GB of saved activations) exceeds the 126 MB L2"},
        "e2e": {"value": tokens / (ms_e2e / args.steps / 1e3), "unit": "tokens/s",
                "h2d_bytes_per_step": per_rank * seq * 4, "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / args.steps,
                "result": "first gradient element after the all-reduce (the gradients stay on the device)"},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": KERNEL_OF_CLASS[dom_name], "achieved": ach, "peak": peak,
                     "unit": "TFLOP/s", "frac": ach / peak, "peak_burst": pk["tflops_burst"],
                     "frac_burst": ach / pk["tflops_burst"],
                     "traffic": traffic_from_profiles("c3", KERNEL_OF_CLASS[dom_name])[0] if args.batch == 0 else None,
                     "peak_source": pk["source"] + " (bf16 matmul, sustained; burst beside it)",
                     "launches": dom["launches"],
                     "whole_step_frac": vjp_flops(cfg, per_rank, seq) / (ms / args.steps / 1e3) / 1e12 / peak,
                     "kernels_ms_per_step": {k: v["ms"] / psteps for k, v in prof.items() if v["launches"]}},
        "clocks": clocks,
    }
    if comm:
        comm.destroy()
    return line


def run_decode(args, rank, world, local, B, dist):
    """Config 5: 7B-shape decode, batch 64, 4096 cached tokens per sequence, one token per step."""
    cfg, dname, batch, ctx0, desc = WORKLOADS["c5"]
    if args.batch > 0:
        batch = args.batch
        desc += f" [batch overridden to {batch}]"
    dev = torch.device("cuda", local)
    pk = peaks()
    tp = world
    steps_total = 128
    cfg = dict(cfg, seq_len=ctx0 + steps_total)
    if args.layers > 0:
        cfg = dict(cfg, n_layers=args.layers)
        desc += f" [layers overridden to {args.layers}]"
    comm = B.Comm(rank, world) if tp > 1 else None
    page = 128
    max_pages = (ctx0 + steps_total + page - 1) // page
    n_pages = batch * max_pages
    plan = B.Plan(cfg, torch.bfloat16, tp_rank=rank, tp_size=tp, comm=comm)
    # weights first (leaves + packed copy live together only here), then the cache:
    # at tp=1 the cache is 141.7 GB and the packed weights 13.2 GB of the 180 GB
    w = synth_weights(cfg, torch.bfloat16, dev)
    plan.pack_weights(w)
    torch.cuda.synchronize()
    del w
    torch.cuda.empty_cache()
    kv = plan.new_kv_pages(n_pages, page)
    g = torch.Generator(device=dev).manual_seed(400 + rank)
    for l in range(cfg["n_layers"]):
        kv[l].normal_(0.0, 1.0, generator=g)
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, max_pages).contiguous()
    gen = torch.Generator().manual_seed(500)
    host_tok = torch.randint(0, cfg["vocab_size"], (batch,), generator=gen, dtype=torch.int32).pin_memory()
    dev_tok = host_tok.to(dev)
    tok_stage = torch.empty(batch, dtype=torch.int32, device=dev)
    logits = torch.empty(batch, plan.vocab_local, dtype=torch.float32, device=dev)
    host_logits = torch.empty(batch, plan.vocab_local, dtype=torch.float32).pin_memory()
    steps = min(args.steps, steps_total - args.warmup)

    def step(i, e2e=False, base=0):
        pos = ctx0 + ((base + i) % steps_total)
        if e2e:
            tok_stage.copy_(host_tok, non_blocking=True)
            plan.decode_step(pos, kv, table, tokens=tok_stage, logits=logits)
            host_logits.copy_(logits, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        else:
            plan.decode_step(pos, kv, table, tokens=dev_tok, logits=logits)

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    l0 = B.launch_count()
    ms = timed(lambda i: step(i, base=args.warmup), steps, world, dist)
    launches = B.launch_count() - l0
    ms_e2e = timed(lambda i: step(i, True, base=args.warmup), steps, world, dist)
    clocks = sampler.stop() if rank == 0 else None
    B.profile_enable(True)
    timed(lambda i: step(i, base=args.warmup), steps, world, dist)
    prof = B.profile_read()
    B.profile_enable(False)
    if B.device_status() != 0:
        raise RuntimeError("device status word set during the timed region")
    L, d, h, V = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
    W = L * (4 * d * d + 3 * d * h) + V * d
    ctx_avg = ctx0 + args.warmup + steps / 2.0
    bytes_step = (W * 2 + 2 * ctx_avg * d * 2 * L * batch) / tp  # weights once + K and V once, per GPU
    att = prof["attention_decode"]
    ach = att["work"] / (att["ms"] / 1e3) / 1e9 if att["ms"] > 0 else 0.0
    value = batch / (ms / steps / 1e3)
    line = {
        "metric": "tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "batch": batch, "context": ctx0, "parallelism": f"tp{tp}",
                   "l2_policy": "each step streams the whole KV cache and all weights (>100 GB), far above L2"},
        "e2e": {"value": batch / (ms_e2e / steps / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": batch * 4,
                "d2h_bytes_per_step": batch * plan.vocab_local * 4, "ms_per_step": ms_e2e / steps,
                "result": "logits of the new token of every sequence"},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": KERNEL_OF_CLASS["attention_decode"], "achieved": ach,
                     "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
                     "traffic": traffic_from_profiles("c5", KERNEL_OF_CLASS["attention_decode"])[0]
                     if args.batch == 0 and args.layers == 0 else None,
                     "peak_source": pk["source"] + " (copy bandwidth)", "launches": att["launches"],
                     "whole_step_frac": bytes_step / (ms / steps / 1e3) / 1e9 / pk["hbm_gbs"],
                     "kernels_ms_per_step": {k: v["ms"] / steps for k, v in prof.items() if v["launches"]}},
        "clocks": clocks,
    }
    if comm:
        comm.destroy()
    return line


def claim_stdout():
    """Keeps a private handle on the real standard output for the one JSON line and points file descriptor 1 at
    standard error, so that whatever libraries print (NCCL_DEBUG=INFO writes to stdout) cannot split the line."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


def main():
    real_stdout = claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tune-tp", action="store_true",
                    help="tensor parallel: time both exchange schedules before the warm-up and run the faster one")
    ap.add_argument("--batch", type=int, default=0, help="override the batch per rank (profiling on a small case)")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling on a small case)")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            real_stdout.write(json.dumps(line) + "\n")
            real_stdout.flush()
        return
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    import b200_llama as B

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        if args.workload in ("c1", "c2", "c4"):
            line = run_prefill(args, rank, world, local, B, dist)
        elif args.workload == "c3":
            line = run_vjp(args, rank, world, local, B, dist)
        else:
            line = run_decode(args, rank, world, local, B, dist)
    finally:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
    if rank == 0 and line is not None:
        real_stdout.write(json.dumps(line) + "\n")
        real_stdout.flush()


if __name__ == "__main__":
    main()
