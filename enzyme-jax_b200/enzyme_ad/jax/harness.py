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
  here: all three rows time the same kernel sequence and are measured
  separately.  As in the reference, ``revprimal`` chooses between the call that
  also returns the primal result (``splatvjp``, test/test_utils.py:499-505) and
  the one that returns the cotangents only (``splatvjp_noprim``, :508-514; the
  reference's llama test sets ``revprimal = False``, test/llama.py:311);
* the reverse rows differentiate with respect to EVERY input of the call, as
  the reference does: ``(x, weights, key_cache, value_cache)`` for the
  reference's own call shape, the weights for the token-sequence shape;
* results are cross-checked like the reference's ``recursive_check``
  (test/test_utils.py:522-550, :678-681) against a baseline the caller passes
  (there, the first pipeline; here, e.g. the CPU oracle), leaf by leaf with
  ``atol`` / ``rtol`` (1e-3 in the reference's llama test);
* the ``Forward`` row (``jax.jvp(fn, ins, dins)`` in the reference, test/test_utils.py:689-735) is timed when
  tangents ``dins`` are passed: ``(dx, dweights, d_key_cache, d_value_cache)`` for the reference's own call shape, a
  dict of weight-leaf tangents for the token-sequence shape;
* times are CUDA-event times on the launching stream, not profiler traces.
"""
from __future__ import annotations

import csv
import os
from typing import Callable, Dict, List, Optional

import torch

from .primitives import _LlamaRoute, vjp

CSV_HEADER = ["Benchmark Name", "Pass Pipeline", "Backend", "Key", "Time"]
REVERSE_KEYS = ("PreRev", "PostRev", "BothRev")


def recursive_check(tester, lhs, rhs, pname=None) -> None:
    """Leaf-by-leaf comparison of two result trees (dicts, lists / tuples, tensors, None) with the tester's
    ``atol`` / ``rtol``; raises ``AssertionError`` naming the first leaf that differs (test/test_utils.py:522-550)."""

    def walk(a, b, path):
        if a is None and b is None:
            return
        if isinstance(a, dict):
            assert isinstance(b, dict) and sorted(a) == sorted(b), f"{pname}: keys differ at {path or 'root'}"
            for k in a:
                walk(a[k], b[k], f"{path}.{k}" if path else str(k))
            return
        if isinstance(a, (list, tuple)):
            assert isinstance(b, (list, tuple)) and len(a) == len(b), f"{pname}: lengths differ at {path or 'root'}"
            for i, (x, y) in enumerate(zip(a, b)):
                walk(x, y, f"{path}[{i}]")
            return
        x = torch.as_tensor(a).detach().double().cpu()
        y = torch.as_tensor(b).detach().double().cpu()
        assert x.shape == y.shape, f"{pname}: shapes differ at {path or 'root'}: {tuple(x.shape)} vs {tuple(y.shape)}"
        if not torch.allclose(x, y, atol=tester.atol, rtol=tester.rtol):
            err = float((x - y).abs().max())
            raise AssertionError(f"{tester.__class__.__name__} {pname}: leaf {path or 'root'} differs, max error {err:.3e} "
                                 f"(atol {tester.atol}, rtol {tester.rtol})")

    walk(lhs, rhs, "")


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
        self.atol = 1e-3
        self.rtol = 1e-3

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

    def harness(self, name: str, fn: Callable, ins, douts: Optional[torch.Tensor] = None, *, dins=None,
                baseline_primal=None, baseline_grads=None, baseline_tangent=None) -> Dict[str, float]:
        """Times ``fn`` (a decorated llama function) on ``ins`` and cross-checks its results.

        ``ins`` is ``(x, weights, key_cache, value_cache)`` -- the reference's own call -- or ``(tokens, weights)``.
        With a cotangent ``douts`` of the result the three reverse rows are timed too, differentiating with respect
        to every input; with tangents ``dins`` of the weight leaves (token-sequence shape) the ``Forward`` row.
        ``baseline_primal`` / ``baseline_tangent`` / ``baseline_grads`` (the trees another implementation produced for
        the same inputs) are compared with ours by ``recursive_check``.  Returns ``{key: seconds}``.
        """
        route: _LlamaRoute = getattr(fn, "_b200_route", None)
        if route is None:
            raise NotImplementedError("harness needs a function decorated with enzyme_jax_ir(pipeline_options=B200Pipeline(...))")
        out: Dict[str, float] = {}
        primal = fn(*ins)  # packs the weights, creates the plan
        if baseline_primal is not None:
            recursive_check(self, primal, baseline_primal, "Primal")
        out["Primal"] = self._avg_seconds(lambda: fn(*ins))
        self.pretty_print_table(name, self.pipeline_name, self.backend, "Primal", out["Primal"])
        if dins is not None and len(ins) == 4:
            # the reference's call: dins = (dx, dweights, d_key_cache, d_value_cache), as test/llama.py:316
            x, weights, kc, vc = ins
            dx, dweights, dkc, dvc = dins
            plan = route._ensure(weights, False)
            _, tangent = plan.token_jvp(x, kc, vc, dx, dweights, dkc, dvc)
            if baseline_tangent is not None:
                recursive_check(self, tangent, baseline_tangent, "Forward")
            out["Forward"] = self._avg_seconds(lambda: plan.token_jvp(x, kc, vc, dx, dweights, dkc, dvc))
            self.pretty_print_table(name, self.pipeline_name, self.backend, "Forward", out["Forward"])
        elif dins is not None:
            plan = route._ensure(ins[1], False)
            _, tangent = plan.forward_jvp(ins[0], dins)
            if baseline_tangent is not None:
                recursive_check(self, tangent, baseline_tangent, "Forward")
            out["Forward"] = self._avg_seconds(lambda: plan.forward_jvp(ins[0], dins))
            self.pretty_print_table(name, self.pipeline_name, self.backend, "Forward", out["Forward"])
        if douts is None:
            return out
        result, pullback = vjp(fn, *ins)
        grads = pullback(douts)
        if baseline_grads is not None:
            recursive_check(self, grads, baseline_grads, "Reverse")
        if len(ins) == 4:
            x, weights, kc, vc = ins
            plan = route._ensure(weights, True)

            def reverse():  # primal and cotangents: token_vjp returns the hidden state along with them
                plan.token_vjp(x, kc, vc, douts)

            reverse_noprim = reverse  # one fused call either way: the primal costs nothing extra to return
        else:
            tokens, weights = ins
            plan = route._ensure(weights, True)
            tok = tokens.to(plan.device, torch.int32).contiguous()
            dlog = douts.to(plan.device, torch.float32).contiguous()
            saved, packed = plan.new_saved(*tok.shape), plan.new_grads()

            def reverse():
                # revprimal: the primal result is produced along with the gradients
                plan.forward(tok, saved=saved)
                plan.backward(tok, dlog, saved, packed)

            def reverse_noprim():
                plan.backward(tok, dlog, saved, packed)

            plan.forward(tok, saved=saved)
        call = reverse if self.revprimal else reverse_noprim
        for key in REVERSE_KEYS:
            out[key] = self._avg_seconds(call)
            self.pretty_print_table(name, self.pipeline_name, self.backend, key, out[key])
        return out


class Llama(EnzymeJaxTest):
    """The reference's ``test/llama.py`` class name, so that the default output
    file is ``results_Llama.csv`` as there (``test/test_utils.py:600-601``), with
    that test's settings (``revprimal = False``, ``atol = rtol = 1e-3``,
    test/llama.py:311-319)."""

    def __init__(self, repeat: int = 50, warmup: int = 3):
        super().__init__(repeat, warmup)
        self.revprimal = False
