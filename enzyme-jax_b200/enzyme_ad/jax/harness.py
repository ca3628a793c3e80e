"""Timing harness with the reference test suite's output format.

The reference times every benchmark through ``EnzymeJaxTest.harness``
(``test/test_utils.py:626-887``) and writes one row per (pipeline, backend, key)
to ``results_<ClassName>.csv`` with the header ``Benchmark Name, Pass Pipeline,
Backend, Key, Time`` (``test/test_utils.py:589-614``); the keys are ``Primal``,
``Forward``, ``PreRev``, ``PostRev`` and ``BothRev``, the time is the average
seconds per call over ``repeat`` calls (50 by default).

This class produces the same rows for a function decorated with
``enzyme_jax_ir(pipeline_options=B200Pipeline(...))`` so that the numbers drop
into whatever reads the reference's CSV files.  What differs, by construction:

* one pipeline (``B200``) and one backend (``gpu``);
* ``PreRev`` / ``PostRev`` / ``BothRev`` name the place of the AD pass relative
  to the optimisation passes of a compiler pipeline.  There is no pass pipeline
  here: all three rows time the same kernel sequence (forward keeping the
  activations, then the backward pass), and are measured separately;
* no ``Forward`` (JVP) row: forward mode is not built;
* times are CUDA-event times on the launching stream, not profiler traces.
"""
from __future__ import annotations

import csv
import os
from typing import Callable, Dict, List, Optional

import torch

from .primitives import _LlamaRoute

CSV_HEADER = ["Benchmark Name", "Pass Pipeline", "Backend", "Key", "Time"]
REVERSE_KEYS = ("PreRev", "PostRev", "BothRev")


class EnzymeJaxTest:
    """Same attributes and method names as the reference's base class where they
    apply (``repeat``, ``results``, ``pretty_print_table``, ``write_results_csv``,
    ``harness``); it is not a ``unittest`` case."""

    pipeline_name = "B200"
    backend = "gpu"

    def __init__(self, repeat: int = 50, warmup: int = 3):
        self.repeat = int(repeat)
        self.warmup = int(warmup)
        self.results: List[str] = []
        self.revprimal = True

    # -- output ---------------------------------------------------------------
    def pretty_print_table(self, name, pname, backend, key, time):
        print("{:<20}\t{:<20}\t{:<15}\t{:<10}\t{:<15.8f}".format(name, pname, backend, key, time), flush=True)
        self.results.append("{}\t{}\t{}\t{}\t{}".format(name, pname, backend, key, time))

    def write_results_csv(self, filename: str = "") -> str:
        if filename == "":
            filename = f"results_{self.__class__.__name__}.csv"
        outfile = os.path.join(os.environ.get("TEST_UNDECLARED_OUTPUTS_DIR", "."), filename)
        with open(outfile, "w", newline="") as f:
            writer = csv.writer(f)
            writer.writerow(CSV_HEADER)
            for line in self.results:
                writer.writerow(line.split("\t"))
        print(f"Results written to {outfile}")
        return outfile

    # -- timing ---------------------------------------------------------------
    def _avg_seconds(self, call: Callable[[], None]) -> float:
        for _ in range(self.warmup):
            call()
        stream = torch.cuda.current_stream()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record(stream)
        for _ in range(self.repeat):
            call()
        t1.record(stream)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) * 1e-3 / self.repeat

    def harness(self, name: str, fn: Callable, ins, douts: Optional[torch.Tensor] = None) -> Dict[str, float]:
        """Times ``fn`` (a decorated llama function) on ``ins``.

        ``ins`` is ``(x, weights, key_cache, value_cache)`` -- the reference's own
        call, Primal row only -- or ``(tokens, weights)``; with a logits cotangent
        ``douts`` the three reverse rows are timed too.  Returns ``{key: seconds}``.
        """
        route: _LlamaRoute = getattr(fn, "_b200_route", None)
        if route is None:
            raise NotImplementedError("harness needs a function decorated with enzyme_jax_ir(pipeline_options=B200Pipeline(...))")
        out: Dict[str, float] = {}
        fn(*ins)  # packs the weights, creates the plan
        out["Primal"] = self._avg_seconds(lambda: fn(*ins))
        self.pretty_print_table(name, self.pipeline_name, self.backend, "Primal", out["Primal"])
        if douts is None:
            return out
        if len(ins) != 2:
            raise NotImplementedError("reverse mode is built for the (tokens, weights) call")
        tokens, weights = ins
        plan = route._ensure(weights, True)
        tok = tokens.to(plan.device, torch.int32).contiguous()
        dlog = douts.to(plan.device, torch.float32).contiguous()
        saved, grads = plan.new_saved(*tok.shape), plan.new_grads()

        def reverse():
            # revprimal: the primal result is produced along with the gradients
            plan.forward(tok, saved=saved)
            plan.backward(tok, dlog, saved, grads)

        def reverse_noprim():
            plan.backward(tok, dlog, saved, grads)

        plan.forward(tok, saved=saved)
        call = reverse if self.revprimal else reverse_noprim
        for key in REVERSE_KEYS:
            out[key] = self._avg_seconds(call)
            self.pretty_print_table(name, self.pipeline_name, self.backend, key, out[key])
        return out


class Llama(EnzymeJaxTest):
    """The reference's ``test/llama.py`` class name, so that the default output
    file is ``results_Llama.csv`` as there (``test/test_utils.py:600-601``)."""
