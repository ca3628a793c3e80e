"""Recognises the llama forward in StableHLO text and rewrites it to the library's custom calls.

The reference hands the StableHLO text of the decorated function to its pass pipeline
(src/enzyme_ad/jax/primitives.py:593-601) and lets passes outline what a library can do into
``stablehlo.custom_call`` operations (Passes/CuDNNHLOOpt.cpp:112-125 outlines dot_general + elementwise clusters,
Passes/LowerEnzymeXLABLAS.cpp:419-479 emits the typed-FFI call with ``backend_config``, layouts and aliases).  This
module is the same step for the one function this build serves, written against the TEXT (there is no MLIR here):

1. ``parse_module`` reads the operations of ``@main`` into a small def-use graph (result, op name, operands,
   attribute text, result type); it understands the pretty form JAX prints and nothing of MLIR beyond that.
2. ``match_llama_forward`` finds the clusters of the reference's ``forward`` (test/llama.py:35-238) by dataflow, not
   by position: RMSNorm (``dot_general(v, v)`` -> divide -> add eps -> sqrt -> reciprocal -> two multiplies,
   test/llama.py:6-10), the seven projections of a layer (a ``dot_general`` whose left operand is a layer slice of a
   rank-3 argument), the pair rotation (a batched ``dot_general`` with a constant table, :161-168), the cache append
   (``concatenate`` of a cache slice with the new row, :170-175), one softmax per head (``reduce`` with ``maximum`` ->
   subtract -> exponential -> sum -> divide, :13-18), SwiGLU (negate -> exponential -> add 1 -> reciprocal, :21-28) and
   the two residual adds.  From them it derives the config (dim, hidden_dim, n_layers, n_heads, cache rows, eps, the
   rotation base) and which ARGUMENT plays which role - so it works on the text after JAX's dead-argument
   elimination too (``wcls`` is unused by the reference's forward and may be absent, primitives.py:1550-1569).
   Anything that does not fit raises ``MatchError``: no partial rewrite.
3. ``rewrite_to_custom_calls`` returns a module with the same signature whose body is two typed-FFI custom calls:
   ``@enzymejax_b200_llama_pack`` (the twelve leaves in the library's order; leaves the function does not have - the
   embedding table, a dropped ``wcls`` - are zero constants, as the reference materialises dropped arguments,
   primitives.py:487-499) and ``@enzymejax_b200_llama_token_fwd`` (x, packed weights, both caches -> hidden state and a
   scratch result, the way the reference appends an ``i8[tmpBuf]`` result, primitives.py:712-727).
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


class MatchError(ValueError):
    pass


@dataclass
class Op:
    result: str
    name: str                 # e.g. "dot_general", "slice", "constant"
    operands: List[str]
    attrs: str                # the text between the operands and the type signature
    shape: Tuple[int, ...]
    line: str


@dataclass
class Module:
    args: List[Tuple[str, Tuple[int, ...]]]     # (%argN, shape)
    ops: Dict[str, Op]
    order: List[str]
    ret: str
    header: List[str] = field(default_factory=list)
    users: Dict[str, List[str]] = field(default_factory=dict)


_TENSOR = re.compile(r"tensor<((?:\d+x)*)(f32|bf16|f16|f64|i32|i8|i1)>")


def _shape_of(type_text: str) -> Tuple[int, ...]:
    m = _TENSOR.search(type_text)
    if not m:
        raise MatchError(f"no tensor type in {type_text!r}")
    dims = m.group(1)
    return tuple(int(d) for d in dims.split("x") if d)


def parse_module(text: str) -> Module:
    lines = text.splitlines()
    sig = next((l for l in lines if "func.func" in l and "@main" in l), None)
    if sig is None:
        raise MatchError("no @main function")
    arg_part = sig[sig.index("(") + 1:]
    args = [(m.group(1), _shape_of(m.group(2))) for m in re.finditer(r"(%arg\d+): (tensor<[^>]*>)", arg_part.split(") ->")[0])]
    mod = Module(args=args, ops={}, order=[], ret="", header=[sig])
    for line in lines:
        s = line.strip()
        if s.startswith("return "):
            mod.ret = re.search(r"(%[\w#]+)", s).group(1)
            continue
        m = re.match(r"(%[\w]+) = stablehlo\.(\w+)(.*)$", s)
        if not m:
            continue
        res, name, rest = m.group(1), m.group(2), m.group(3)
        # the type signature follows the LAST " : " that is outside brackets
        depth, cut = 0, -1
        for i, ch in enumerate(rest):
            if ch in "<[({":
                depth += 1
            elif ch in ">])}":
                depth -= 1
            elif ch == ":" and depth == 0 and rest[i - 1:i + 2] == " : ":
                cut = i
        if cut < 0:
            raise MatchError(f"cannot find the type of {s!r}")
        body, types = rest[:cut], rest[cut + 1:]
        result_type = types.split("->")[-1]
        body_wo_dense = re.sub(r"dense<.*>", "dense<>", body)
        operands = re.findall(r"%[\w]+", body_wo_dense)
        op = Op(res, name, operands, body, _shape_of(result_type), s)
        mod.ops[res] = op
        mod.order.append(res)
        for o in operands:
            mod.users.setdefault(o, []).append(res)
    if not mod.ret:
        raise MatchError("no return")
    return mod


# ---- graph helpers -----------------------------------------------------------------------------------------------

def _through(mod: Module, v: str, names=("reshape", "broadcast_in_dim")) -> str:
    """Follows v backwards through shape-only ops."""
    while v in mod.ops and mod.ops[v].name in names:
        v = mod.ops[v].operands[0]
    return v


def _layer_slice(mod: Module, v: str) -> Optional[Tuple[str, int]]:
    """(argument, layer index) when v is `arg[l, ...]` (slice of the leading dimension + reshape), else None."""
    v = _through(mod, v, ("reshape",))
    if v in mod.ops and mod.ops[v].name == "slice":
        src = mod.ops[v].operands[0]
        if src.startswith("%arg"):
            m = re.search(r"\[(\d+):(\d+)", mod.ops[v].attrs)
            if m and int(m.group(2)) == int(m.group(1)) + 1:
                return src, int(m.group(1))
    return None


def _const_value(mod: Module, v: str) -> Optional[float]:
    v = _through(mod, v)
    if v in mod.ops and mod.ops[v].name == "constant" and mod.ops[v].shape == ():
        m = re.search(r"dense<([-+0-9.eEinfa]+)>", mod.ops[v].attrs)
        if m:
            return float(m.group(1).replace("inf", "inf"))
    return None


def _is(mod: Module, v: str, name: str) -> bool:
    return v in mod.ops and mod.ops[v].name == name


@dataclass
class LlamaMatch:
    config: Dict[str, int]
    pos: int
    rms_eps: float
    rope_theta: Optional[float]
    arg_roles: Dict[str, str]          # "%argN" -> "x" | leaf name | "key_cache" | "value_cache"
    result: str
    clusters: Dict[str, int]           # how many of each cluster were recognised


def _match_rmsnorm(mod: Module, out: str) -> Optional[Tuple[str, str, float]]:
    """out = (gain * v) * broadcast(1 / sqrt(dot(v, v) / n + eps)): returns (v, gain source, eps)."""
    if not _is(mod, out, "multiply"):
        return None
    a, b = mod.ops[out].operands
    for scaled, fac in ((a, b), (b, a)):
        f = _through(mod, fac)
        if not _is(mod, f, "divide"):
            continue
        one, root = mod.ops[f].operands
        if _const_value(mod, one) != 1.0 or not _is(mod, _through(mod, root), "sqrt"):
            continue
        add = mod.ops[_through(mod, root)].operands[0]
        if not _is(mod, add, "add"):
            continue
        mean, eps_v = mod.ops[add].operands
        eps = _const_value(mod, eps_v)
        if eps is None or not _is(mod, mean, "divide"):
            continue
        dot, n_v = mod.ops[mean].operands
        if not _is(mod, dot, "dot_general") or mod.ops[dot].operands[0] != mod.ops[dot].operands[1]:
            continue
        v = mod.ops[dot].operands[0]
        n = _const_value(mod, n_v)
        if not _is(mod, scaled, "multiply") or n is None:
            continue
        g0, g1 = mod.ops[scaled].operands
        gain = g0 if g1 == v else (g1 if g0 == v else None)
        if gain is None or int(n) != (mod.ops[v].shape[0] if v in mod.ops else dict(mod.args)[v][0]):
            continue
        return v, gain, eps
    return None


def match_llama_forward(text: str) -> LlamaMatch:
    mod = parse_module(text)
    shapes = dict(mod.args)
    roles: Dict[str, str] = {}

    def shape(v):
        return mod.ops[v].shape if v in mod.ops else shapes[v]

    # ---- projections: dot_general(layer slice of a rank-3 argument, vector) ---------------------------------
    proj: Dict[Tuple[str, int], str] = {}          # (arg, layer) -> dot op
    for r in mod.order:
        op = mod.ops[r]
        if op.name != "dot_general" or len(op.operands) != 2 or "batching_dims" in op.attrs:
            continue
        ls = _layer_slice(mod, op.operands[0])
        if ls and len(shapes[ls[0]]) == 3 and "contracting_dims = [1] x [0]" in op.attrs:
            if ls in proj:
                raise MatchError(f"{ls[0]} layer {ls[1]} is used by two projections")
            proj[ls] = r
    if not proj:
        raise MatchError("no weight projections found")
    n_layers = 1 + max(l for _, l in proj)
    weight_args = sorted({a for a, _ in proj})
    for a in weight_args:
        if shapes[a][0] != n_layers or any((a, l) not in proj for l in range(n_layers)):
            raise MatchError(f"{a} is not used once per layer")

    # ---- final RMSNorm is the result; walk the layers backwards from it -----------------------------------------
    fin = _match_rmsnorm(mod, mod.ret)
    if fin is None:
        raise MatchError("the result is not an RMSNorm")
    x_last, gain_fin, eps = fin
    if not gain_fin.startswith("%arg") or len(shapes[gain_fin]) != 1:
        raise MatchError("the final gain is not a rank-1 argument")
    roles[gain_fin] = "rms_final_weight"
    dim = shapes[gain_fin][0]

    counts = {"rmsnorm": 1, "projection": 0, "rotation": 0, "cache_append": 0, "softmax": 0, "swiglu": 0, "residual": 0}
    n_heads = None
    hidden = None
    pos = None
    theta = None
    x = x_last
    for l in reversed(range(n_layers)):
        # x = x_mid + w2[l] @ (silu(w1[l] @ xb2) * (w3[l] @ xb2))
        if not _is(mod, x, "add"):
            raise MatchError(f"layer {l}: no residual add after the feed-forward block")
        x_mid, ffn = mod.ops[x].operands
        if not _is(mod, ffn, "dot_general"):
            x_mid, ffn = ffn, x_mid
        ls2 = _layer_slice(mod, mod.ops[ffn].operands[0]) if _is(mod, ffn, "dot_general") else None
        if not ls2 or ls2[1] != l:
            raise MatchError(f"layer {l}: the feed-forward output is not a projection of this layer")
        roles.setdefault(ls2[0], "w2")
        hb = mod.ops[ffn].operands[1]
        if not _is(mod, hb, "multiply"):
            raise MatchError(f"layer {l}: no gate * up product")
        sil, up = mod.ops[hb].operands
        def is_silu(v):
            # v = g * (1 / (1 + exp(-g)))
            if not _is(mod, v, "multiply"):
                return None
            a, b = mod.ops[v].operands
            for g, s in ((a, b), (b, a)):
                if _is(mod, s, "divide") and _is(mod, mod.ops[s].operands[1], "add"):
                    add = mod.ops[s].operands[1]
                    e = [o for o in mod.ops[add].operands if _is(mod, o, "exponential")]
                    if e and _is(mod, mod.ops[e[0]].operands[0], "negate") and mod.ops[mod.ops[e[0]].operands[0]].operands[0] == g:
                        return g
            return None
        gate = is_silu(sil)
        if gate is None:
            gate, up = is_silu(up), sil
        if gate is None or not _is(mod, gate, "dot_general") or not _is(mod, up, "dot_general"):
            raise MatchError(f"layer {l}: SwiGLU not recognised")
        counts["swiglu"] += 1
        lg, lu = _layer_slice(mod, mod.ops[gate].operands[0]), _layer_slice(mod, mod.ops[up].operands[0])
        if not lg or not lu or lg[1] != l or lu[1] != l:
            raise MatchError(f"layer {l}: gate / up are not projections of this layer")
        roles.setdefault(lg[0], "w1")
        roles.setdefault(lu[0], "w3")
        hidden = shapes[lg[0]][1]
        xb2 = mod.ops[gate].operands[1]
        if mod.ops[up].operands[1] != xb2:
            raise MatchError(f"layer {l}: gate and up read different inputs")
        n2 = _match_rmsnorm(mod, xb2)
        if n2 is None or n2[0] != x_mid:
            raise MatchError(f"layer {l}: the feed-forward input is not RMSNorm of the residual stream")
        gl = _layer_slice(mod, n2[1])
        if not gl or gl[1] != l:
            raise MatchError(f"layer {l}: feed-forward gain is not a layer slice")
        roles.setdefault(gl[0], "rms_ffn_weight")
        counts["rmsnorm"] += 1
        counts["projection"] += 3
        counts["residual"] += 1
        # x_mid = x_in + wo[l] @ concat(heads)
        if not _is(mod, x_mid, "add"):
            raise MatchError(f"layer {l}: no residual add after the attention block")
        x_in, att_out = mod.ops[x_mid].operands
        if not _is(mod, att_out, "dot_general"):
            x_in, att_out = att_out, x_in
        lo = _layer_slice(mod, mod.ops[att_out].operands[0]) if _is(mod, att_out, "dot_general") else None
        if not lo or lo[1] != l:
            raise MatchError(f"layer {l}: the attention output is not a projection of this layer")
        roles.setdefault(lo[0], "wo")
        counts["projection"] += 1
        counts["residual"] += 1
        cat = mod.ops[att_out].operands[1]
        if not _is(mod, cat, "concatenate"):
            raise MatchError(f"layer {l}: head outputs are not concatenated")
        heads = [_through(mod, h, ("reshape",)) for h in mod.ops[cat].operands]
        if n_heads is None:
            n_heads = len(heads)
        if len(heads) != n_heads or dim % n_heads:
            raise MatchError(f"layer {l}: {len(heads)} heads, expected {n_heads}")
        hs = dim // n_heads
        kcache = vcache = qrot = None
        for h_i, ho in enumerate(heads):
            # out_h = V[:, head] contracted with softmax(K[:, head] q_h / sqrt(hs))
            if not _is(mod, ho, "dot_general"):
                raise MatchError(f"layer {l} head {h_i}: no value contraction")
            vs, p = mod.ops[ho].operands
            if not _is(mod, p, "divide"):
                raise MatchError(f"layer {l} head {h_i}: probabilities are not a quotient")
            e, ssum = mod.ops[p].operands
            if not _is(mod, _through(mod, e), "exponential"):
                raise MatchError(f"layer {l} head {h_i}: no exponential")
            sub = mod.ops[_through(mod, e)].operands[0]
            if not _is(mod, sub, "subtract") or not _is(mod, _through(mod, mod.ops[sub].operands[1]), "reduce") or \
                    "maximum" not in mod.ops[_through(mod, mod.ops[sub].operands[1])].attrs:
                raise MatchError(f"layer {l} head {h_i}: no max-shifted softmax")
            counts["softmax"] += 1
            scaled = mod.ops[sub].operands[0]
            if not _is(mod, scaled, "divide"):
                raise MatchError(f"layer {l} head {h_i}: scores are not divided by sqrt(head_size)")
            sc = _const_value(mod, mod.ops[scaled].operands[1])
            if sc is None or abs(sc - math.sqrt(hs)) > 1e-4 * math.sqrt(hs):
                raise MatchError(f"layer {l} head {h_i}: score scale {sc}, expected sqrt({hs})")
            scores = mod.ops[scaled].operands[0]
            if not _is(mod, scores, "dot_general"):
                raise MatchError(f"layer {l} head {h_i}: no key contraction")
            ks, qh = mod.ops[scores].operands
            for slc, which in ((ks, "k"), (vs, "v")):
                if not _is(mod, slc, "slice") or not _is(mod, mod.ops[slc].operands[0], "concatenate"):
                    raise MatchError(f"layer {l} head {h_i}: {which} is not a head slice of the appended cache")
                c = mod.ops[slc].operands[0]
                if which == "k":
                    kcache = kcache or c
                    if c != kcache:
                        raise MatchError(f"layer {l}: heads read different key caches")
                else:
                    vcache = vcache or c
                    if c != vcache:
                        raise MatchError(f"layer {l}: heads read different value caches")
            qsrc = mod.ops[qh].operands[0] if _is(mod, qh, "slice") else qh
            qrot = qrot or qsrc
            if qsrc != qrot:
                raise MatchError(f"layer {l}: heads read different queries")
        # the caches: concat(cache[l], new row)
        def cache_parts(c, what):
            old, new = mod.ops[c].operands
            ls = _layer_slice(mod, old)
            if not ls or ls[1] != l or len(shapes[ls[0]]) != 3:
                raise MatchError(f"layer {l}: the {what} cache is not a layer slice of an argument")
            return ls[0], _through(mod, new, ("reshape",))
        karg, knew = cache_parts(kcache, "key")
        varg, vnew = cache_parts(vcache, "value")
        roles.setdefault(karg, "key_cache")
        roles.setdefault(varg, "value_cache")
        counts["cache_append"] += 2
        pos = shapes[karg][1]
        # rotation: batched dot_general of a constant [d/2, 2, 2] table with the pair view of q and k
        def unrotate(v, what):
            v = _through(mod, v, ("reshape",))
            if not _is(mod, v, "dot_general") or "batching_dims = [0] x [0]" not in mod.ops[v].attrs:
                raise MatchError(f"layer {l}: {what} is not rotated by a batched 2x2 product")
            table, pairs = mod.ops[v].operands
            if not _is(mod, table, "constant") or mod.ops[table].shape != (dim // 2, 2, 2):
                raise MatchError(f"layer {l}: the rotation table of {what} is not a constant [dim/2, 2, 2]")
            counts["rotation"] += 1
            return _through(mod, pairs, ("reshape",)), table
        kproj, ktable = unrotate(knew, "k")
        qproj, _ = unrotate(qrot, "q")
        vproj = vnew
        nonlocal_theta = _theta_from_table(mod.ops[ktable].attrs, hs, pos)
        theta = theta if theta is not None else nonlocal_theta
        xb = None
        for pr, role in ((qproj, "wq"), (kproj, "wk"), (vproj, "wv")):
            ls = _layer_slice(mod, mod.ops[pr].operands[0]) if _is(mod, pr, "dot_general") else None
            if not ls or ls[1] != l:
                raise MatchError(f"layer {l}: {role} projection not found")
            roles.setdefault(ls[0], role)
            if roles[ls[0]] != role:
                raise MatchError(f"{ls[0]} plays {roles[ls[0]]} and {role}")
            xb = xb or mod.ops[pr].operands[1]
            if mod.ops[pr].operands[1] != xb:
                raise MatchError(f"layer {l}: q, k, v read different inputs")
        counts["projection"] += 3
        n1 = _match_rmsnorm(mod, xb)
        if n1 is None or n1[0] != x_in:
            raise MatchError(f"layer {l}: the attention input is not RMSNorm of the residual stream")
        ga = _layer_slice(mod, n1[1])
        if not ga or ga[1] != l:
            raise MatchError(f"layer {l}: attention gain is not a layer slice")
        roles.setdefault(ga[0], "rms_att_weight")
        counts["rmsnorm"] += 1
        if abs(n1[2] - eps) > 1e-12 or abs(n2[2] - eps) > 1e-12:
            raise MatchError("the RMSNorm epsilons differ")
        x = x_in
    if not x.startswith("%arg") or shapes[x] != (dim,):
        raise MatchError("the residual stream does not start at a rank-1 argument")
    roles[x] = "x"
    # what is left: wcls (unused by the reference's forward) when it survived dead-argument elimination
    vocab = None
    for a, s in mod.args:
        if a not in roles:
            if len(s) == 2 and s[1] == dim and a not in mod.users:
                roles[a] = "wcls"
                vocab = s[0]
            else:
                raise MatchError(f"argument {a} {s} has no role in the llama forward")
    expect = {"x", "rms_att_weight", "rms_ffn_weight", "rms_final_weight", "w1", "w2", "w3", "wk", "wo", "wq", "wv",
              "key_cache", "value_cache"}
    have = set(roles.values()) - {"wcls"}
    if have != expect:
        raise MatchError(f"roles missing: {sorted(expect - have)}")
    cfg = dict(dim=dim, hidden_dim=hidden, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_heads,
               vocab_size=vocab if vocab is not None else 0)
    return LlamaMatch(config=cfg, pos=pos, rms_eps=eps, rope_theta=theta, arg_roles=roles, result=mod.ret, clusters=counts)


def _theta_from_table(attrs: str, hs: int, pos: int) -> Optional[float]:
    """The rotation base from the constant table: pair j of a head has angle pos * theta^(-2j/hs)
    (test/llama.py:129-135); None when the table does not determine it (pos == 0 or one pair per head)."""
    nums = [float(t) for t in re.findall(r"-?\d+\.\d+e[-+]\d+|-?\d+\.\d+", attrs)]
    if pos == 0 or hs < 4 or len(nums) < 8:
        return None
    c1, s1 = nums[4], nums[6]          # second pair: [[cos, -sin], [sin, cos]]
    ang = math.atan2(s1, c1)
    if ang <= 0:
        return None
    return (pos / ang) ** (hs / 2.0)


# ---- rewrite -------------------------------------------------------------------------------------------------------

LEAF_ORDER = ("rms_att_weight", "rms_ffn_weight", "rms_final_weight", "token_embedding_table", "w1", "w2", "w3", "wcls",
              "wk", "wo", "wq", "wv")


def _ttype(shape, et="f32"):
    return "tensor<" + "".join(f"{d}x" for d in shape) + et + ">"


def rewrite_to_custom_calls(text: str, *, vocab_size: Optional[int] = None, seq_len: Optional[int] = None,
                            sizes=None) -> str:
    """The module of `text` with its body replaced by the library's typed-FFI custom calls.  ``vocab_size`` is needed
    when ``wcls`` was dropped from the signature; ``seq_len`` (default: cache rows + 1) bounds the rotation table of the
    plan; ``sizes(config, pos) -> {"packed_bytes", "token_workspace_bytes"}`` defaults to the library's
    ``b200_static_sizes``."""
    m = match_llama_forward(text)
    mod = parse_module(text)
    shapes = dict(mod.args)
    cfg = dict(m.config)
    if not cfg["vocab_size"]:
        if vocab_size is None:
            raise MatchError("wcls is not among the arguments: pass vocab_size")
        cfg["vocab_size"] = int(vocab_size)
    cfg["seq_len"] = int(seq_len) if seq_len else m.pos + 1
    if sizes is None:
        import torch
        import b200_llama
        sizes = lambda c, p: b200_llama.static_sizes(c, torch.float32, False, p, m.rope_theta or 10000.0, m.rms_eps)
    sz = sizes(cfg, m.pos)
    by_role = {r: a for a, r in m.arg_roles.items()}
    L, d, h, V = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
    leaf_shapes = {"rms_att_weight": (L, d), "rms_ffn_weight": (L, d), "rms_final_weight": (d,),
                   "token_embedding_table": (V, d), "w1": (L, h, d), "w2": (L, d, h), "w3": (L, h, d), "wcls": (V, d),
                   "wk": (L, d, d), "wo": (L, d, d), "wq": (L, d, d), "wv": (L, d, d)}
    body = []
    operands = []
    for leaf in LEAF_ORDER:
        if leaf in by_role:
            if shapes[by_role[leaf]] != leaf_shapes[leaf]:
                raise MatchError(f"{leaf} has shape {shapes[by_role[leaf]]}, expected {leaf_shapes[leaf]}")
            operands.append(by_role[leaf])
        else:  # a leaf the function does not have: zeros (its value cannot reach the result)
            name = f"%zero_{leaf}"
            body.append(f"    {name} = stablehlo.constant dense<0.000000e+00> : {_ttype(leaf_shapes[leaf])}")
            operands.append(name)
    attrs = (f"dim = {d} : i32, hidden_dim = {h} : i32, n_layers = {L} : i32, n_heads = {cfg['n_heads']} : i32, "
             f"n_kv_heads = {cfg['n_kv_heads']} : i32, vocab_size = {V} : i32, seq_len = {cfg['seq_len']} : i32, "
             f"dtype = 0 : i32, rope_theta = {m.rope_theta or 10000.0:.6e} : f32, rms_eps = {m.rms_eps:.6e} : f32")

    def layouts(shs):
        return "[" + ", ".join("dense<[" + ", ".join(str(i) for i in reversed(range(len(s)))) + "]> : tensor<" +
                               f"{len(s)}xindex>" for s in shs) + "]"

    pk_shapes = [leaf_shapes[l] for l in LEAF_ORDER]
    packed_t = _ttype((sz["packed_bytes"],), "i8")
    body.append(
        f"    %packed = stablehlo.custom_call @enzymejax_b200_llama_pack({', '.join(operands)}) "
        f"{{api_version = 4 : i32, backend_config = {{{attrs}, with_transposed = false}}, "
        f"operand_layouts = {layouts(pk_shapes)}, result_layouts = {layouts([(sz['packed_bytes'],)])}}} : "
        f"({', '.join(_ttype(s) for s in pk_shapes)}) -> {packed_t}")
    x, kc, vc = by_role["x"], by_role["key_cache"], by_role["value_cache"]
    ws_t = _ttype((sz["token_workspace_bytes"],), "i8")
    in_shapes = [(d,), (sz["packed_bytes"],), shapes[kc], shapes[vc]]
    in_types = [_ttype((d,)), packed_t, _ttype(shapes[kc]), _ttype(shapes[vc])]
    body.append(
        f"    %out:2 = stablehlo.custom_call @enzymejax_b200_llama_token_fwd({x}, %packed, {kc}, {vc}) "
        f"{{api_version = 4 : i32, backend_config = {{{attrs}}}, operand_layouts = {layouts(in_shapes)}, "
        f"result_layouts = {layouts([(d,), (sz['token_workspace_bytes'],)])}}} : "
        f"({', '.join(in_types)}) -> ({_ttype((d,))}, {ws_t})")
    body.append(f"    return %out#0 : {_ttype((d,))}")
    lines = text.splitlines()
    i_sig = next(i for i, l in enumerate(lines) if "func.func" in l and "@main" in l)
    return "\n".join(lines[:i_sig + 1] + body + ["  }", "}"]) + "\n"
