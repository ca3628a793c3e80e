"""The C-ABI library loads without a GPU and exports every symbol the header
declares; argument checks that precede any CUDA call answer with status codes."""
import ctypes
import os
import re

import pytest

import b200_llama as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200_llama.h")).read()
    return sorted(set(re.findall(r"B200_API[^;(]*?\b(b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    lib = B.lib()
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(B.EXPORTS) == names


def test_version_and_error_string():
    lib = B.lib()
    assert lib.b200_version() == b"0.1"
    assert lib.b200_plan_create(None, 0, 1, None, None) == 1
    assert b"null" in lib.b200_last_error()


def test_null_arguments_are_rejected_before_any_launch():
    lib = B.lib()
    n = ctypes.c_size_t(0)
    assert lib.b200_packed_weight_bytes(None, 0, ctypes.byref(n)) == 1
    assert lib.b200_workspace_bytes(None, 0, 1, 1, ctypes.byref(n)) == 1
    assert lib.b200_gemm(None, None, None, 1, 16, 16, 16, 16, 16, 0, 0, 1, 1, 0, 0, None) == 1
    assert lib.b200_comm_unique_id(None) == 1
    assert lib.b200_backward(None, None, 1, 1, None, None, None, None, 0, None, 0, None) == 1


def test_plan_needs_a_device():
    import pytest
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError):
        B.Plan(dict(dim=64, hidden_dim=128, n_layers=1, n_heads=2, n_kv_heads=2, vocab_size=96, seq_len=8))


def test_python_surface_has_the_reference_names():
    import enzyme_ad.jax as EJ
    import pytest
    # src/enzyme_ad/jax/__init__.py:1-12 of the reference
    for name in ("cpp_call", "ffi_call", "hlo_call", "enzyme_jax_ir", "XLAPipeline", "JaXPipeline", "optimize_module",
                 "export", "full_optimization_pass_pipeline", "optimization_passes"):
        assert hasattr(EJ, name), name
    assert EJ.JaXPipeline("a,enzyme-wrap{x},b,enzyme-wrap{y}").ad_level() == 2
    assert EJ.XLAPipeline("n").export_llvm() == "n" and EJ.XLAPipeline().mlir_ad() is False
    for fn in (EJ.cpp_call, EJ.hlo_call, EJ.optimize_module, EJ.export, EJ.optimization_passes):
        with pytest.raises(NotImplementedError):
            fn()
    with pytest.raises(NotImplementedError):
        EJ.enzyme_jax_ir()(lambda x: x)


def test_harness_csv_format_matches_reference(tmp_path, monkeypatch):
    """Header and row layout of test/test_utils.py:589-614, without a GPU."""
    import csv
    from enzyme_ad.jax.harness import CSV_HEADER, Llama
    h = Llama()
    assert h.repeat == 50
    h.pretty_print_table("llama", "B200", "gpu", "Primal", 0.00125)
    monkeypatch.setenv("TEST_UNDECLARED_OUTPUTS_DIR", str(tmp_path))
    path = h.write_results_csv()
    rows = list(csv.reader(open(path)))
    assert path.endswith("results_Llama.csv")
    assert rows[0] == ["Benchmark Name", "Pass Pipeline", "Backend", "Key", "Time"] == CSV_HEADER
    assert rows[1] == ["llama", "B200", "gpu", "Primal", "0.00125"]


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` times the CPU restatement of the path and prints one JSON line with the keys the
    measurement contract names; it needs no GPU."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "tokens_per_second" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["n_gpus"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"]


def test_page_allocator_host_logic():
    a = B.PageAllocator(6)
    x = a.alloc(4)
    assert sorted(x) == x and len(set(x)) == 4 and a.free_pages == 2
    a.free([x[1], x[2]])
    y = a.alloc(3)
    assert len(set(y) | {x[0], x[3]}) == 5 and a.free_pages == 1
    with pytest.raises(B.B200Error):
        a.alloc(2)                                   # exhausted
    with pytest.raises(B.B200Error):
        a.free([a.alloc(1)[0], 99])                  # not a page of this pool


def test_ffi_registration_entry_points_and_python_glue(monkeypatch):
    """The library always exports the three FFI functions; in a build without the XLA FFI headers they say so.  The
    Python glue wraps every handler address in a PyCapsule named for XLA and hands it to jax.ffi.register_ffi_target:
    checked against a stand-in for jax.ffi and a stand-in library that has handlers."""
    import ctypes
    import enzyme_ad.jax.primitives as P
    lib = B.lib()
    if not lib.b200_ffi_available():
        assert lib.b200_ffi_handler(b"enzymejax_b200_llama_fwd") is None
        assert lib.registerEnzymeJaXB200FFI() == 10      # B200_ERR_UNSUPPORTED
        with pytest.raises(NotImplementedError):
            P.register_ffi_targets(jax_ffi=object())

    class FakeLib:
        def b200_ffi_available(self):
            return 1

        def b200_ffi_handler(self, name):
            return 0x1000 + len(name)   # any non-null address

    class FakeJaxFfi:
        def __init__(self):
            self.calls = []

        def register_ffi_target(self, name, capsule, platform=None, **kw):
            self.calls.append((name, capsule, platform))

    monkeypatch.setattr(P._B, "lib", lambda: FakeLib())
    monkeypatch.setattr(P, "_FFI_REGISTERED", False)
    fake = FakeJaxFfi()
    names = P.register_ffi_targets(jax_ffi=fake)
    assert [c[0] for c in fake.calls] == list(names) and len(names) == 8
    assert all(c[2] == "CUDA" for c in fake.calls)
    get_name = ctypes.pythonapi.PyCapsule_GetName
    get_name.restype = ctypes.c_char_p
    get_name.argtypes = [ctypes.py_object]
    assert all(get_name(c[1]) == b"xla._CUSTOM_CALL_TARGET" for c in fake.calls)
    P.register_ffi_targets(jax_ffi=fake)          # idempotent
    assert len(fake.calls) == 8


def test_static_sizes_need_no_device():
    import torch
    cfg = dict(dim=288, hidden_dim=768, n_layers=6, n_heads=6, n_kv_heads=6, vocab_size=32000, seq_len=256)
    s32 = B.static_sizes(cfg, torch.float32, False, 1)
    s16 = B.static_sizes(cfg, torch.bfloat16, True, 1)
    n_params = 6 * (4 * 288 * 288 + 3 * 288 * 768) + 2 * 32000 * 288
    assert s32["packed_bytes"] >= 4 * n_params and s32["packed_bytes"] < 4 * n_params + 64 * 1024
    assert s16["packed_bytes"] > 2 * 2 * (n_params - 32000 * 288)   # bf16, with transposed copies of the matrices
    assert s32["grad_bytes"] == s32["packed_bytes"] and s32["token_workspace_bytes"] > 0
