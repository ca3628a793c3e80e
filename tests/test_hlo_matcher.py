"""The StableHLO-text matcher of the llama forward (enzyme_ad/jax/hlo_matcher.py) on the committed fixtures: text of
the reference's own ``forward`` source traced into StableHLO (tests/golden/make_stablehlo.py), with and without the
argument JAX's dead-argument elimination drops.  CPU only."""
import os
import re
import subprocess
import sys

import pytest

from enzyme_ad.jax import hlo_matcher as M

HERE = os.path.dirname(os.path.abspath(__file__))
FULL = open(os.path.join(HERE, "golden", "llama_forward_tiny.stablehlo.mlir")).read()
DCE = open(os.path.join(HERE, "golden", "llama_forward_tiny_dce.stablehlo.mlir")).read()
TINY = dict(dim=8, hidden_dim=16, n_layers=2, n_heads=2, n_kv_heads=2)


def test_fixture_is_recognised_with_config_roles_and_constants():
    m = M.match_llama_forward(FULL)
    assert {k: m.config[k] for k in TINY} == TINY and m.config["vocab_size"] == 32
    assert m.pos == 2 and abs(m.rms_eps - 1e-5) < 1e-12 and abs(m.rope_theta - 10000.0) < 1.0
    # arguments in JAX's flattening order: x, sorted weight leaves, the caches
    order = ["x", "rms_att_weight", "rms_ffn_weight", "rms_final_weight", "w1", "w2", "w3", "wcls", "wk", "wo", "wq", "wv",
             "key_cache", "value_cache"]
    assert [m.arg_roles[f"%arg{i}"] for i in range(14)] == order
    L, H = 2, 2
    assert m.clusters == {"rmsnorm": 2 * L + 1, "projection": 7 * L, "rotation": 2 * L, "cache_append": 2 * L,
                          "softmax": L * H, "swiglu": L, "residual": 2 * L}


def test_roles_come_from_dataflow_not_position():
    """After dead-argument elimination wcls is gone and every later argument moves up by one."""
    m = M.match_llama_forward(DCE)
    assert m.config["vocab_size"] == 0 and "wcls" not in m.arg_roles.values()
    assert m.arg_roles["%arg7"] == "wk" and m.arg_roles["%arg11"] == "key_cache" and m.arg_roles["%arg12"] == "value_cache"
    # renaming SSA values and swapping two commutative operands changes nothing
    t = re.sub(r"%(\d+)\b", lambda g: f"%v{int(g.group(1)) + 1000}", FULL)
    t = re.sub(r"stablehlo\.multiply (%v\d+), (%arg0) ", r"stablehlo.multiply \2, \1 ", t, count=1)
    assert M.match_llama_forward(t).arg_roles == M.match_llama_forward(FULL).arg_roles


def test_rewrite_emits_typed_ffi_custom_calls_with_library_sizes():
    import torch
    import b200_llama as B
    out = M.rewrite_to_custom_calls(DCE, vocab_size=32, seq_len=16)
    sig_in = [l for l in DCE.splitlines() if "func.func" in l][0]
    assert sig_in in out                                       # same signature
    calls = re.findall(r"stablehlo\.custom_call @(\w+)", out)
    assert calls == ["enzymejax_b200_llama_pack", "enzymejax_b200_llama_token_fwd"]
    assert out.count("api_version = 4 : i32") == 2 and "backend_config = {dim = 8 : i32" in out
    assert "%zero_wcls = stablehlo.constant dense<0.000000e+00> : tensor<32x8xf32>" in out   # dropped leaf -> zeros
    sz = B.static_sizes(dict(TINY, vocab_size=32, seq_len=16), torch.float32, False, 2)
    assert f"-> tensor<{sz['packed_bytes']}xi8>" in out
    assert f"tensor<{sz['token_workspace_bytes']}xi8>)" in out
    assert "return %out#0 : tensor<8xf32>" in out
    # the leaves reach the pack call in the library's order
    pack = [l for l in out.splitlines() if "llama_pack" in l][0]
    ops = re.search(r"llama_pack\(([^)]*)\)", pack).group(1).split(", ")
    assert ops == ["%arg1", "%arg2", "%arg3", "%zero_token_embedding_table", "%arg4", "%arg5", "%arg6", "%zero_wcls", "%arg7",
                   "%arg8", "%arg9", "%arg10"]
    with pytest.raises(M.MatchError):
        M.rewrite_to_custom_calls(DCE)                           # vocabulary unknown without wcls


@pytest.mark.parametrize("what", ["scale", "softmax", "residual", "silu", "extra_arg", "eps"])
def test_functions_that_are_not_the_llama_forward_are_refused(what):
    t = FULL
    if what == "scale":        # scores divided by something other than sqrt(head_size)
        t = t.replace("dense<2.000000e+00> : tensor<f32>", "dense<3.000000e+00> : tensor<f32>", 1)
    elif what == "softmax":    # no max shift
        i = t.index("stablehlo.subtract")
        t = t[:i] + "stablehlo.add" + t[i + len("stablehlo.subtract"):]
    elif what == "residual":   # the last residual add replaced by a product
        i = t.rindex("stablehlo.add")
        t = t[:i] + "stablehlo.multiply" + t[i + len("stablehlo.add"):]
    elif what == "silu":       # exp(x) instead of exp(-x)
        i = t.index("stablehlo.negate")
        t = t[:i] + "stablehlo.abs" + t[i + len("stablehlo.negate"):]
    elif what == "extra_arg":  # an argument with no role
        t = t.replace("%arg13: tensor<2x2x8xf32>)", "%arg13: tensor<2x2x8xf32>, %arg14: tensor<5xf32>)")
    elif what == "eps":        # different epsilons in two norms
        i = t.rindex("dense<1.000000e-05>")
        t = t[:i] + "dense<2.000000e-05>" + t[i + len("dense<1.000000e-05>"):]
    with pytest.raises(M.MatchError):
        M.match_llama_forward(t)


def test_fixture_regenerates_from_the_reference_source():
    """With the reference tree at hand (B200_REFERENCE_ROOT), the generator reproduces the committed fixtures."""
    root = os.environ.get("B200_REFERENCE_ROOT")
    if not root or not os.path.exists(os.path.join(root, "test", "llama.py")):
        pytest.skip("B200_REFERENCE_ROOT is not set")
    sys.path.insert(0, os.path.join(HERE, "golden"))
    import make_stablehlo
    assert make_stablehlo.emit(root, drop_unused=False) == FULL
    assert make_stablehlo.emit(root, drop_unused=True) == DCE
