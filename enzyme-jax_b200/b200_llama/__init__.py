"""Host-side driver of the B200 llama path.

Thin ``ctypes`` layer over ``libb200_llama.so`` (the C ABI declared in
``include/b200_llama.h``).  PyTorch supplies device memory, streams and
``torch.distributed``; every computation runs in the library's own sm_100a
kernels.  There is no CPU fallback: loading fails loudly when the library has
not been built, and every entry point raises :class:`B200Error` on a non-zero
status.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, byref, c_char_p, c_float, c_int32, c_size_t, c_uint32, c_void_p
from typing import Dict, Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libb200_llama.so")

F32, BF16 = 0, 1
LEAF_ORDER = (
    "rms_att_weight", "rms_ffn_weight", "rms_final_weight", "token_embedding_table",
    "w1", "w2", "w3", "wcls", "wk", "wo", "wq", "wv",
)
CONFIG_KEYS = ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "seq_len")

EXPORTS = (
    "b200_last_error", "b200_version", "b200_device_status", "b200_plan_create", "b200_plan_destroy",
    "b200_packed_weight_bytes", "b200_pack_weights", "b200_workspace_bytes", "b200_saved_bytes", "b200_forward",
    "b200_backward", "b200_packed_grad_bytes", "b200_unpack_grads", "b200_allreduce_f32", "b200_decode_step",
    "b200_gemm", "b200_rmsnorm", "b200_attention", "b200_comm_unique_id", "b200_comm_init_rank",
    "b200_comm_destroy", "b200_launch_count", "b200_profile_enable", "b200_profile_read",
    "b200_attention_decode_scratch_bytes", "b200_attention_decode", "b200_attention_decode_static",
    "b200_attention_backward", "b200_comm_peer_memory", "b200_selftest_bounded_wait", "b200_argmax",
    "b200_selftest_peer_wait", "b200_plan_cached", "b200_ffi_available", "b200_ffi_handler",
    "b200_token_vjp_workspace_bytes", "b200_token_vjp", "b200_comm_init_rank_ex", "b200_comm_setup_peer_memory",
    "b200_comm_attach_memory", "b200_tp_exchange_buffers", "b200_tp_reduce_norm", "b200_token_forward",
    "b200_static_sizes", "b200_jvp_workspace_bytes", "b200_forward_jvp", "b200_token_jvp_workspace_bytes",
    "b200_token_jvp", "b200_plan_set_option", "b200_plan_get_option",
)


class B200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"b200 status {status}: {message}")
        self.status = status


class _Config(ctypes.Structure):
    _fields_ = [(k, c_int32) for k in CONFIG_KEYS] + [("dtype", c_int32), ("rope_theta", c_float), ("rms_eps", c_float)]


_lib = None


def lib() -> ctypes.CDLL:
    """Loads the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is None:
        path = os.environ.get("B200_LLAMA_LIB", LIB_PATH)  # another build of the same ABI, e.g. to compare two kernels
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python enzyme-jax_b200/build.py` "
                "(there is no fallback implementation)")
        l = ctypes.CDLL(path)
        l.b200_last_error.restype = c_char_p
        l.b200_version.restype = c_char_p
        for name in EXPORTS:
            fn = getattr(l, name)
            if name not in ("b200_last_error", "b200_version", "b200_ffi_handler"):
                fn.restype = c_int32
        l.b200_ffi_handler.restype = c_void_p
        l.b200_ffi_handler.argtypes = [c_char_p]
        l.registerEnzymeJaXB200FFI.restype = c_int32
        l.b200_plan_cached.argtypes = [POINTER(_Config), c_int32, c_int32, c_void_p, POINTER(c_void_p)]
        l.b200_selftest_peer_wait.argtypes = [ctypes.c_int64, c_void_p, c_void_p]
        l.b200_token_vjp_workspace_bytes.argtypes = [c_void_p, c_int32, POINTER(c_size_t)]
        l.b200_token_forward.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p,
                                         c_size_t, c_void_p]
        l.b200_jvp_workspace_bytes.argtypes = [c_void_p, c_int32, c_int32, POINTER(c_size_t)]
        l.b200_forward_jvp.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_size_t, c_void_p]
        l.b200_token_jvp_workspace_bytes.argtypes = [c_void_p, c_int32, POINTER(c_size_t)]
        l.b200_token_jvp.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
        l.b200_static_sizes.argtypes = [POINTER(_Config), c_int32, c_int32, POINTER(c_size_t), POINTER(c_size_t),
                                        POINTER(c_size_t)]
        l.b200_token_vjp.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
        l.b200_launch_count.restype = ctypes.c_int64
        l.b200_profile_enable.argtypes = [c_int32]
        l.b200_profile_read.argtypes = [c_int32, POINTER(ctypes.c_double), POINTER(ctypes.c_double),
                                        POINTER(ctypes.c_int64)]
        l.b200_plan_create.argtypes = [POINTER(_Config), c_int32, c_int32, c_void_p, POINTER(c_void_p)]
        l.b200_plan_destroy.argtypes = [c_void_p]
        l.b200_plan_set_option.argtypes = [c_void_p, c_char_p, c_int32]
        l.b200_plan_get_option.argtypes = [c_void_p, c_char_p, POINTER(c_int32)]
        l.b200_packed_weight_bytes.argtypes = [c_void_p, c_int32, POINTER(c_size_t)]
        l.b200_packed_grad_bytes.argtypes = [c_void_p, POINTER(c_size_t)]
        l.b200_pack_weights.argtypes = [c_void_p, POINTER(c_void_p), c_int32, c_int32, c_void_p, c_void_p]
        l.b200_workspace_bytes.argtypes = [c_void_p, c_int32, c_int32, c_int32, POINTER(c_size_t)]
        l.b200_saved_bytes.argtypes = [c_void_p, c_int32, c_int32, POINTER(c_size_t)]
        l.b200_forward.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_size_t, c_void_p]
        l.b200_backward.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int32, c_void_p, c_size_t, c_void_p]
        l.b200_unpack_grads.argtypes = [c_void_p, c_void_p, POINTER(c_void_p), c_void_p]
        l.b200_allreduce_f32.argtypes = [c_void_p, c_void_p, c_size_t, c_void_p]
        l.b200_decode_step.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p,
                                       c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
        l.b200_gemm.argtypes = [c_void_p, c_void_p, c_void_p] + [c_int32] * 12 + [c_void_p]
        l.b200_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_float, c_int32,
                                   c_void_p]
        l.b200_attention.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int32] * 9 + [c_void_p]
        l.b200_attention_decode_scratch_bytes.argtypes = [c_int32] * 4 + [POINTER(c_size_t)]
        l.b200_attention_decode.argtypes = [c_void_p] * 5 + [c_size_t] + [c_int32] * 10 + [c_void_p]
        l.b200_attention_decode_static.argtypes = [c_void_p] * 4 + [c_int32] * 10 + [c_void_p]
        l.b200_attention_backward.argtypes = [c_void_p] * 10 + [c_int32] * 9 + [c_void_p]
        l.b200_selftest_bounded_wait.argtypes = [ctypes.c_int64, c_void_p, c_void_p]
        l.b200_argmax.argtypes = [c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p]
        l.b200_device_status.argtypes = [c_void_p, POINTER(c_uint32)]
        l.b200_comm_unique_id.argtypes = [c_void_p]
        l.b200_comm_init_rank.argtypes = [c_void_p, c_int32, c_int32, POINTER(c_void_p)]
        l.b200_comm_init_rank_ex.argtypes = [c_void_p, c_int32, c_int32, c_int32, POINTER(c_void_p)]
        l.b200_comm_setup_peer_memory.argtypes = [c_void_p]
        l.b200_comm_attach_memory.argtypes = [c_void_p, c_size_t, POINTER(c_void_p), c_void_p]
        l.b200_tp_exchange_buffers.argtypes = [c_void_p, c_size_t, POINTER(c_void_p), POINTER(c_void_p)]
        l.b200_tp_reduce_norm.argtypes = [c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_float,
                                          c_void_p]
        l.b200_comm_destroy.argtypes = [c_void_p]
        l.b200_comm_peer_memory.argtypes = [c_void_p, POINTER(c_int32)]
        _lib = l
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise B200Error(status, lib().b200_last_error().decode("utf-8", "replace"))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise B200Error(3, f"unsupported dtype {dtype}")


def static_sizes(config: Dict[str, int], dtype: torch.dtype = torch.float32, with_transposed: bool = False,
                 pos: int = 0, rope_theta: float = 10000.0, rms_eps: float = 1e-5) -> Dict[str, int]:
    """Byte sizes of the packed weights, the packed gradients and the workspace of the reference-shaped call for a
    model on one GPU, computed without a device (``b200_static_sizes``)."""
    c = _Config(*[int(config[k]) for k in CONFIG_KEYS], _dt(dtype), rope_theta, rms_eps)
    a, b, w = c_size_t(0), c_size_t(0), c_size_t(0)
    check(lib().b200_static_sizes(byref(c), int(with_transposed), pos, byref(a), byref(b), byref(w)))
    return {"packed_bytes": a.value, "grad_bytes": b.value, "token_workspace_bytes": w.value}


def device_status() -> int:
    """Reads and clears the device status word (synchronises the stream)."""
    code = c_uint32(0)
    check(lib().b200_device_status(_stream(), byref(code)))
    return code.value


def launch_count() -> int:
    return int(lib().b200_launch_count())


PROFILE_CLASSES = ("gemm_tcgen05", "gemm_ffma", "attention_fwd", "attention_bwd", "attention_decode", "allreduce",
                   "gemm_tcgen05_pair")


def profile_enable(on: bool) -> None:
    check(lib().b200_profile_enable(int(on)))


def profile_read() -> Dict[str, Dict[str, float]]:
    """Per kernel class: summed ms, summed algorithmic work, launches (synchronises the recorded events)."""
    out = {}
    for i, name in enumerate(PROFILE_CLASSES):
        ms, work, n = ctypes.c_double(0), ctypes.c_double(0), ctypes.c_int64(0)
        check(lib().b200_profile_read(i, byref(ms), byref(work), byref(n)))
        out[name] = {"ms": ms.value, "work": work.value, "launches": int(n.value)}
    return out


# --------------------------------------------------------------------------
# single kernels
# --------------------------------------------------------------------------

def gemm(a: torch.Tensor, b: torch.Tensor, *, ta=False, tb=False, out_dtype=None, impl=0,
         out: Optional[torch.Tensor] = None, accumulate=False) -> torch.Tensor:
    """Y = op(a) @ op(b)^T with fp32 accumulation.  a is [M,K] ([K,M] with ta), b is [N,K] ([K,N] with tb)."""
    M, K = (a.shape[1], a.shape[0]) if ta else (a.shape[0], a.shape[1])
    N = b.shape[1] if tb else b.shape[0]
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    check(lib().b200_gemm(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                          out.stride(0), int(ta), int(tb), _dt(a.dtype), _dt(out.dtype), int(accumulate), impl,
                          _stream()))
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float = 1e-5, out_dtype=torch.float32):
    rows, dim = x.shape
    y = torch.empty(rows, dim, dtype=out_dtype, device=x.device)
    rinv = torch.empty(rows, dtype=torch.float32, device=x.device)
    check(lib().b200_rmsnorm(x.data_ptr(), gain.data_ptr(), y.data_ptr(), rinv.data_ptr(), rows, dim, eps,
                             _dt(out_dtype), _stream()))
    return y, rinv


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, batch: int, seq: int, n_heads: int, impl=0):
    """Causal attention; q,k,v are [batch*seq, n_heads*head_size] (possibly strided row views)."""
    T, d = q.shape
    hs = d // n_heads
    o = torch.empty(T, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(batch, n_heads, seq, dtype=torch.float32, device=q.device)
    check(lib().b200_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), batch, seq,
                               n_heads, hs, q.stride(0), k.stride(0), o.stride(0), _dt(q.dtype), impl, _stream()))
    return o, lse


def attention_backward(qkv: torch.Tensor, o: torch.Tensor, lse: torch.Tensor, d_o: torch.Tensor, batch: int, seq: int,
                       n_heads: int, impl=0) -> torch.Tensor:
    """Backward of causal attention for a packed qkv [batch*seq, 3*d]; returns dqkv of the same shape."""
    T, d3 = qkv.shape
    d = d3 // 3
    es = qkv.element_size()
    dqkv = torch.empty_like(qkv)
    delta = torch.empty(batch * n_heads * seq, dtype=torch.float32, device=qkv.device)
    base, dbase = qkv.data_ptr(), dqkv.data_ptr()
    check(lib().b200_attention_backward(base, base + d * es, base + 2 * d * es, o.data_ptr(), lse.data_ptr(),
                                        d_o.data_ptr(), dbase, dbase + d * es, dbase + 2 * d * es, delta.data_ptr(),
                                        batch, seq, n_heads, d // n_heads, d3, d3, o.stride(0), _dt(qkv.dtype), impl,
                                        _stream()))
    return dqkv


def attention_decode(q: torch.Tensor, kv_layer: torch.Tensor, page_table: torch.Tensor, ctx: int, n_heads: int,
                     scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode attention of q [batch, n_heads*hs] over one layer of a paged cache [2, n_pages, n_heads, page_size, hs]."""
    batch, d = q.shape
    hs = d // n_heads
    n_pages, page_size = kv_layer.shape[1], kv_layer.shape[3]
    o = torch.empty(batch, d, dtype=q.dtype, device=q.device)
    if scratch is None:
        n = c_size_t(0)
        check(lib().b200_attention_decode_scratch_bytes(batch, n_heads, hs, ctx, byref(n)))
        scratch = torch.empty(n.value, dtype=torch.uint8, device=q.device)
    check(lib().b200_attention_decode(q.data_ptr(), kv_layer.data_ptr(), page_table.data_ptr(), o.data_ptr(),
                                      scratch.data_ptr(), scratch.numel(), batch, ctx, n_heads, hs, q.stride(0),
                                      o.stride(0), n_pages, page_size, page_table.shape[1], _dt(q.dtype), _stream()))
    return o


def attention_decode_static(q: torch.Tensor, kv_layer: torch.Tensor, page_table: torch.Tensor, ctx: int,
                            n_heads: int, out: torch.Tensor) -> torch.Tensor:
    """Decode attention that allocates nothing: the caller passes the output, the scratch is the
    library's built-in 4 MiB array.  For callers that cannot allocate device memory (no scratch
    operand to give, fixed memory pool, cudaMalloc not permitted where they run).  Calls that may
    overlap on the GPU race on the shared scratch; make the first call outside stream capture."""
    batch, d = q.shape
    hs = d // n_heads
    check(lib().b200_attention_decode_static(q.data_ptr(), kv_layer.data_ptr(), page_table.data_ptr(),
                                             out.data_ptr(), batch, ctx, n_heads, hs, q.stride(0), out.stride(0),
                                             kv_layer.shape[1], kv_layer.shape[3], page_table.shape[1],
                                             _dt(q.dtype), _stream()))
    return out


# --------------------------------------------------------------------------
# communicator
# --------------------------------------------------------------------------

def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-wise argmax of fp32 logits [rows, cols] on the device (lowest index among equal maxima) -> int32 [rows]."""
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise B200Error(3, "argmax takes fp32 [rows, cols] logits with unit column stride")
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    check(lib().b200_argmax(logits.data_ptr(), logits.shape[0], logits.shape[1], logits.stride(0), out.data_ptr(),
                            _stream()))
    return out


class PageAllocator:
    """Free list over the pages of one KV pool (host side).  Sequences take whole pages; a page table row lists a
    sequence's pages in position order, as ``b200_decode_step`` reads it."""

    def __init__(self, n_pages: int):
        self.n_pages = int(n_pages)
        self._free = list(range(self.n_pages - 1, -1, -1))

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def alloc(self, n: int):
        if n > len(self._free):
            raise B200Error(5, f"KV pool exhausted: {n} pages wanted, {len(self._free)} free")
        return [self._free.pop() for _ in range(n)]

    def free(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages or p in self._free:
                raise B200Error(1, f"page {p} is not an allocated page of this pool")
        self._free.extend(reversed(list(pages)))


def _new_unique_id() -> bytes:
    ident = ctypes.create_string_buffer(128)
    check(lib().b200_comm_unique_id(ident))
    return ident.raw


def share_unique_id(rank: int, world: int, make_id, group=None) -> bytes:
    """Host-side hand-off of the 128-byte communicator id: rank 0 makes it, every rank receives it, and every rank
    then confirms to every other that it is there.  A rank that died or never joined makes the hand-off fail on the
    others within the process group's timeout; that surfaces as ``B200Error`` with the NCCL status code, before any
    GPU work that would wait for the missing rank has been launched."""
    import torch.distributed as dist
    box = [make_id() if rank == 0 else None]
    try:
        dist.broadcast_object_list(box, src=0, group=group)
        present = [None] * world
        dist.all_gather_object(present, rank, group=group)
    except Exception as exc:  # a timeout or a closed connection: some rank is not there
        raise B200Error(8, f"the communicator id did not reach every rank (rank {rank} of {world}): {exc}") from exc
    if sorted(present) != list(range(world)) or not isinstance(box[0], (bytes, bytearray)) or len(box[0]) != 128:
        raise B200Error(8, f"communicator hand-off incomplete: ranks present {present}")
    return bytes(box[0])


class Comm:
    """NCCL communicator created from a unique id that rank 0 shares through
    ``torch.distributed`` (any backend: the id is 128 bytes of host data)."""

    def __init__(self, rank: int, world: int, group=None, symmetric: Optional[bool] = None):
        raw = share_unique_id(rank, world, _new_unique_id, group)
        ident = ctypes.create_string_buffer(raw, 128)
        handle = c_void_p()
        if symmetric is None:
            symmetric = os.environ.get("B200_SYMM_MEM", "1") != "0"
        symmetric = bool(symmetric) and world > 1
        check(lib().b200_comm_init_rank_ex(ident, rank, world, 0 if symmetric else 1, byref(handle)))
        self.handle, self.rank, self.world = handle, rank, world
        self._symm = None
        if symmetric and not self._attach_symmetric(group):
            check(lib().b200_comm_setup_peer_memory(handle))  # the library's own CUDA-IPC buffers instead

    def _attach_symmetric(self, group) -> bool:
        """Exchange memory from torch.distributed's symmetric-memory allocator: one block per rank, mapped into every
        rank, and (on NVSwitch systems) bound to a multicast object, which lets the tensor-parallel exchange reduce
        inside the switch.  Every rank reaches ``b200_comm_attach_memory`` whatever happened before it, so that the
        ranks agree on the outcome; False means that no rank attached."""
        import torch.distributed as dist
        nbytes = (int(os.environ.get("B200_P2P_MB", "136")) << 20) + 4096
        ptrs = (c_void_p * self.world)()
        mc = None
        keep = None
        try:
            import torch.distributed._symmetric_memory as symm_mem
            dev = torch.device("cuda", torch.cuda.current_device())
            block = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
            hdl = symm_mem.rendezvous(block, group=group if group is not None else dist.group.WORLD)
            for r, p in enumerate(hdl.buffer_ptrs):
                ptrs[r] = p
            mc = int(hdl.multicast_ptr) or None
            keep = (block, hdl)
        except Exception:  # no symmetric memory here: attach nothing, but still take part in the agreement
            ptrs = (c_void_p * self.world)()
            mc = None
        status = lib().b200_comm_attach_memory(self.handle, nbytes, ptrs, mc)
        if status == 0:
            self._symm = keep  # the library never frees it; it lives as long as this object
            return True
        if status != 10:
            check(status)
        return False

    def peer_memory(self) -> int:
        """0: tensor-parallel partial sums travel through NCCL; 1: through peer-mapped memory (plain loads and stores
        over NVLink); 2: through peer-mapped memory bound to a multicast object (summed inside the NVLink switch)."""
        on = c_int32(0)
        check(lib().b200_comm_peer_memory(self.handle, byref(on)))
        return int(on.value)

    def exchange_buffers(self, rows_total: int, dim: int, dtype: torch.dtype):
        """(part, gathered): views of this rank's exchange memory, [rows_total, dim] of ``dtype`` each (see
        ``b200_tp_exchange_buffers``).  They alias library-managed device memory: valid while the communicator lives."""
        es = 2 if dtype == torch.bfloat16 else 4
        n = rows_total * dim * es
        part, gath = c_void_p(), c_void_p()
        check(lib().b200_tp_exchange_buffers(self.handle, n, byref(part), byref(gath)))

        def view(ptr):
            class _Raw:  # __cuda_array_interface__ lets torch wrap device memory it does not own
                __cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (ptr.value, False), "version": 2}
            return torch.as_tensor(_Raw(), device="cuda").view(dtype).view(rows_total, dim)

        return view(part), view(gath)

    def reduce_norm(self, rows_total: int, dim: int, dtype: torch.dtype, x_own: torch.Tensor, gain: torch.Tensor,
                    eps: float = 1e-5, reduce: bool = True) -> None:
        check(lib().b200_tp_reduce_norm(self.handle, rows_total, dim, _dt(dtype), int(reduce), x_own.data_ptr(),
                                        gain.data_ptr(), eps, _stream()))

    def allreduce_f32(self, t: torch.Tensor) -> None:
        check(lib().b200_allreduce_f32(self.handle, t.data_ptr(), t.numel(), _stream()))

    def destroy(self) -> None:
        if self.handle:
            check(lib().b200_comm_destroy(self.handle))
            self.handle = None
            self._symm = None


# --------------------------------------------------------------------------
# plan
# --------------------------------------------------------------------------

class Plan:
    """A model on the current CUDA device: config, packed weights, buffers."""

    def __init__(self, config: Dict[str, int], dtype: torch.dtype = torch.bfloat16, *, tp_rank: int = 0,
                 tp_size: int = 1, comm: Optional[Comm] = None, rope_theta: float = 10000.0, rms_eps: float = 1e-5):
        if not torch.cuda.is_available():
            raise RuntimeError("the B200 llama path needs a CUDA device; there is no CPU implementation")
        self.config = dict(config)
        self.dtype = dtype
        self.tp_rank, self.tp_size, self.comm = tp_rank, tp_size, comm
        self.device = torch.device("cuda", torch.cuda.current_device())
        c = _Config(*[int(config[k]) for k in CONFIG_KEYS], _dt(dtype), rope_theta, rms_eps)
        self._h = c_void_p()
        check(lib().b200_plan_create(byref(c), tp_rank, tp_size, comm.handle if comm else None, byref(self._h)))
        self.packed: Optional[torch.Tensor] = None
        self.with_transposed = False
        self._ws: Optional[torch.Tensor] = None
        self._ws_pinned_by_graphs = []  # workspaces that captured graphs point into: kept alive with the plan
        self.vocab_local = config["vocab_size"] // tp_size
        self.d_local = config["dim"] // tp_size

    def close(self) -> None:
        if self._h:
            lib().b200_plan_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- buffers ---------------------------------------------------------
    def _bytes(self, fn, *args) -> int:
        n = c_size_t(0)
        check(fn(self._h, *args, byref(n)))
        return n.value

    def workspace(self, mode: int, batch: int, seq: int) -> torch.Tensor:
        need = self._bytes(lib().b200_workspace_bytes, mode, batch, seq)
        if self._ws is None or self._ws.numel() < need:
            if not any(self._ws is t for t in self._ws_pinned_by_graphs):
                self._ws = None  # free before the larger allocation, unless a captured graph still points into it
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._ws

    def _check_capturable(self) -> None:
        if self.tp_size > 1:
            raise B200Error(10, "a tensor-parallel plan cannot be captured into a CUDA graph: the peer exchange "
                                "numbers its rounds from the host; launch its steps eagerly")

    def saved_bytes(self, batch: int, seq: int) -> int:
        return self._bytes(lib().b200_saved_bytes, batch, seq)

    def grad_bytes(self) -> int:
        return self._bytes(lib().b200_packed_grad_bytes)

    # ---- weights ---------------------------------------------------------
    def pack_weights(self, weights: Dict[str, torch.Tensor], with_transposed: bool = False) -> None:
        """``weights``: the reference's weight dict (full, unsharded leaves) on this device."""
        leaves = []
        dts = set()
        for name in LEAF_ORDER:
            t = weights[name]
            if not t.is_cuda or not t.is_contiguous():
                raise B200Error(1, f"leaf {name} must be a contiguous CUDA tensor")
            leaves.append(t)
            dts.add(t.dtype)
        if len(dts) != 1:
            raise B200Error(3, "all leaves must share one dtype")
        n = self._bytes(lib().b200_packed_weight_bytes, int(with_transposed))
        self.packed = torch.empty(n, dtype=torch.uint8, device=self.device)
        arr = (c_void_p * len(leaves))(*[t.data_ptr() for t in leaves])
        check(lib().b200_pack_weights(self._h, arr, _dt(dts.pop()), int(with_transposed), self.packed.data_ptr(),
                                      _stream()))
        self.with_transposed = with_transposed

    def pack_tangents(self, tangents: Dict[str, torch.Tensor]) -> torch.Tensor:
        """Packs a dict of weight-leaf tangents (same names and shapes as the weights; missing leaves count as zero)
        into the layout of the weights, for ``forward_jvp``."""
        cfg = self.config
        L, d, h, V = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
        shapes = {"rms_att_weight": (L, d), "rms_ffn_weight": (L, d), "rms_final_weight": (d,),
                  "token_embedding_table": (V, d), "w1": (L, h, d), "w2": (L, d, h), "w3": (L, h, d), "wcls": (V, d),
                  "wk": (L, d, d), "wo": (L, d, d), "wq": (L, d, d), "wv": (L, d, d)}
        leaves = []
        for name in LEAF_ORDER:
            t = tangents.get(name)
            t = torch.zeros(shapes[name], dtype=self.dtype, device=self.device) if t is None else \
                t.to(self.device, self.dtype).contiguous()
            if tuple(t.shape) != shapes[name]:
                raise B200Error(2, f"tangent of {name} has shape {tuple(t.shape)}, expected {shapes[name]}")
            leaves.append(t)
        n = self._bytes(lib().b200_packed_weight_bytes, 0)
        packed = torch.empty(n, dtype=torch.uint8, device=self.device)
        arr = (c_void_p * len(leaves))(*[t.data_ptr() for t in leaves])
        check(lib().b200_pack_weights(self._h, arr, _dt(self.dtype), 0, packed.data_ptr(), _stream()))
        return packed

    def forward_jvp(self, tokens: torch.Tensor, tangents: Dict[str, torch.Tensor]):
        """``jax.jvp``-shaped: returns ``(logits, dlogits)`` for the tangents of the weight leaves."""
        B, S = tokens.shape
        tok = tokens.to(self.device, torch.int32).contiguous()
        saved = self.new_saved(B, S)
        logits = self.forward(tok, saved=saved)
        packed_dw = self.pack_tangents(tangents)
        dlogits = torch.empty(B, S, self.vocab_local, dtype=torch.float32, device=self.device)
        need = self._bytes(lib().b200_jvp_workspace_bytes, B, S)
        ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        check(lib().b200_forward_jvp(self._h, tok.data_ptr(), B, S, self.packed.data_ptr(), packed_dw.data_ptr(),
                                     saved.data_ptr(), dlogits.data_ptr(), ws.data_ptr(), ws.numel(), _stream()))
        return logits, dlogits

    # ---- run-time options -------------------------------------------------
    def set_option(self, name: str, value: int) -> None:
        """Sets a run-time option of the plan (``b200_plan_set_option``), e.g. ``"tp_pipeline"``; every rank of a
        tensor-parallel plan must set the same value."""
        check(lib().b200_plan_set_option(self._h, name.encode(), int(value)))

    def get_option(self, name: str) -> int:
        v = c_int32(0)
        check(lib().b200_plan_get_option(self._h, name.encode(), byref(v)))
        return int(v.value)

    def tune_tensor_parallel(self, tokens: torch.Tensor, logits: Optional[torch.Tensor] = None, reps: int = 2,
                             group=None) -> Dict[str, float]:
        """Times the tensor-parallel prefill of ``tokens`` both ways - one batch with the exchange between the
        kernels, and two halves with the exchange of one beside the compute of the other - and keeps the faster one
        (``"tp_pipeline"``).  Which one wins depends on the rank count and on the NVLink fabric of the moment, so it is
        measured, during warm-up, and not assumed.  Collective: every rank calls it with the same shapes; the ranks
        agree through a MAX all-reduce of their device times over ``group`` (default: the world group), so they all
        keep the same choice.  Returns the two times in ms and the choice."""
        if self.tp_size < 2:
            return {"one_batch_ms": 0.0, "two_halves_ms": 0.0, "tp_pipeline": 0}
        import torch.distributed as dist
        times = []
        for mode in (0, 1):
            self.set_option("tp_pipeline", mode)
            self.forward(tokens, logits=logits)  # first call of a variant: kernel attributes, workspace
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            dist.barrier(group=group)
            a.record()
            for _ in range(reps):
                self.forward(tokens, logits=logits)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) / reps)
        t = torch.tensor(times, dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        one, two = float(t[0]), float(t[1])
        choice = 1 if two < one else 0
        self.set_option("tp_pipeline", choice)
        return {"one_batch_ms": one, "two_halves_ms": two, "tp_pipeline": choice}

    # ---- forward / backward ---------------------------------------------
    def forward(self, tokens: torch.Tensor, *, saved: Optional[torch.Tensor] = None,
                kv_out: Optional[torch.Tensor] = None, logits: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens int32 [B,S] on the device -> fp32 logits [B,S,V/tp]."""
        B, S = tokens.shape
        if tokens.dtype != torch.int32 or not tokens.is_cuda:
            raise B200Error(3, "tokens must be an int32 CUDA tensor")
        if logits is None:
            logits = torch.empty(B, S, self.vocab_local, dtype=torch.float32, device=self.device)
        ws = self.workspace(1 if saved is not None else 0, B, S)
        check(lib().b200_forward(self._h, tokens.data_ptr(), B, S, self.packed.data_ptr(), logits.data_ptr(),
                                 _ptr(saved), _ptr(kv_out), ws.data_ptr(), ws.numel(), _stream()))
        return logits

    def capture_forward(self, tokens: torch.Tensor, logits: torch.Tensor) -> "torch.cuda.CUDAGraph":
        """Captures one forward over fixed token / logits buffers into a CUDA graph (the kernel sequence of a
        plan is static, so a replay costs one launch instead of 1 + 7L + 2).  Run one eager forward first so that
        the workspace exists and every kernel attribute is set outside the capture.  The graph points into the plan's
        workspace of this moment, which the plan keeps alive from here on even when a later, larger call replaces it."""
        self._check_capturable()
        self.forward(tokens, logits=logits)
        torch.cuda.synchronize()
        self._ws_pinned_by_graphs.append(self._ws)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.forward(tokens, logits=logits)
        return graph

    def capture_prefill_step(self, host_tokens: torch.Tensor, tokens: torch.Tensor, logits: torch.Tensor,
                             last_logits: torch.Tensor, host_last_logits: torch.Tensor) -> "torch.cuda.CUDAGraph":
        """One serving step as a single CUDA graph: upload `host_tokens` (pinned) into `tokens`, run the forward,
        gather the last-position logits of every sequence into `last_logits` and copy them to
        `host_last_logits` (pinned).  Copies inside the graph keep consecutive replays back to back; separate
        copy calls between replays cost more than the copies themselves."""
        if not (host_tokens.is_pinned() and host_last_logits.is_pinned()):
            raise B200Error(1, "host buffers of a captured step must be pinned")
        self._check_capturable()
        self.forward(tokens, logits=logits)
        torch.cuda.synchronize()
        self._ws_pinned_by_graphs.append(self._ws)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            tokens.copy_(host_tokens, non_blocking=True)
            self.forward(tokens, logits=logits)
            last_logits.copy_(logits[:, -1, :])
            host_last_logits.copy_(last_logits, non_blocking=True)
        return graph

    def new_saved(self, batch: int, seq: int) -> torch.Tensor:
        return torch.empty(self.saved_bytes(batch, seq), dtype=torch.uint8, device=self.device)

    def new_grads(self) -> torch.Tensor:
        return torch.zeros(self.grad_bytes() // 4, dtype=torch.float32, device=self.device)

    def backward(self, tokens: torch.Tensor, dlogits: torch.Tensor, saved: torch.Tensor, grads: torch.Tensor,
                 accumulate: bool = False) -> torch.Tensor:
        if not self.with_transposed:
            raise B200Error(1, "backward needs weights packed with with_transposed=True")
        B, S = tokens.shape
        ws = self.workspace(2, B, S)
        check(lib().b200_backward(self._h, tokens.data_ptr(), B, S, self.packed.data_ptr(), dlogits.data_ptr(),
                                  saved.data_ptr(), grads.data_ptr(), int(accumulate), ws.data_ptr(), ws.numel(),
                                  _stream()))
        return grads

    def unpack_grads(self, grads: torch.Tensor) -> Dict[str, torch.Tensor]:
        cfg = self.config
        L, d, h, V = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
        shapes = {
            "rms_att_weight": (L, d), "rms_ffn_weight": (L, d), "rms_final_weight": (d,),
            "token_embedding_table": (V, d), "w1": (L, h, d), "w2": (L, d, h), "w3": (L, h, d), "wcls": (V, d),
            "wk": (L, d, d), "wo": (L, d, d), "wq": (L, d, d), "wv": (L, d, d),
        }
        out = {k: torch.empty(shapes[k], dtype=torch.float32, device=self.device) for k in LEAF_ORDER}
        arr = (c_void_p * len(LEAF_ORDER))(*[out[k].data_ptr() for k in LEAF_ORDER])
        check(lib().b200_unpack_grads(self._h, grads.data_ptr(), arr, _stream()))
        return out

    def token_forward(self, x: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor) -> torch.Tensor:
        """The reference's call over flat caches: ``forward(x, weights, key_cache, value_cache) -> hidden`` with
        ``x`` fp32 [d] and caches [L, pos, d]."""
        L, d = self.config["n_layers"], self.config["dim"]
        pos = int(key_cache.shape[1])
        if tuple(key_cache.shape) != (L, pos, d) or tuple(value_cache.shape) != (L, pos, d):
            raise B200Error(2, f"caches must be [{L}, pos, {d}], got {tuple(key_cache.shape)} and {tuple(value_cache.shape)}")
        dev = self.device
        xin = x.to(dev, torch.float32).reshape(d).contiguous()
        kc = key_cache.to(dev, self.dtype).contiguous()
        vc = value_cache.to(dev, self.dtype).contiguous()
        hidden = torch.empty(d, dtype=torch.float32, device=dev)
        need = self._bytes(lib().b200_token_vjp_workspace_bytes, pos)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        check(lib().b200_token_forward(self._h, xin.data_ptr(), kc.data_ptr() if pos else None,
                                       vc.data_ptr() if pos else None, pos, self.packed.data_ptr(), hidden.data_ptr(),
                                       ws.data_ptr(), ws.numel(), _stream()))
        return hidden

    def token_jvp(self, x, key_cache, value_cache, dx, dweights: Dict[str, torch.Tensor], d_key_cache, d_value_cache):
        """Forward mode of the reference's own call with tangents for all of its inputs (``jax.jvp(fn, ins, dins)``).
        Returns ``(hidden, d_hidden)``, both fp32 [d]."""
        L, d = self.config["n_layers"], self.config["dim"]
        pos = int(key_cache.shape[1])
        for name, c in (("key_cache", key_cache), ("value_cache", value_cache), ("d_key_cache", d_key_cache),
                        ("d_value_cache", d_value_cache)):
            if tuple(c.shape) != (L, pos, d):
                raise B200Error(2, f"{name} must be [{L}, {pos}, {d}], got {tuple(c.shape)}")
        dev = self.device
        f32 = lambda t: t.to(dev, torch.float32).reshape(d).contiguous()
        cd = lambda t: t.to(dev, self.dtype).contiguous()
        xin, dxin = f32(x), f32(dx)
        kc, vc, dkc, dvc = cd(key_cache), cd(value_cache), cd(d_key_cache), cd(d_value_cache)
        packed_dw = self.pack_tangents(dweights)
        hidden = torch.empty(d, dtype=torch.float32, device=dev)
        d_hidden = torch.empty(d, dtype=torch.float32, device=dev)
        need = self._bytes(lib().b200_token_jvp_workspace_bytes, pos)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        ptr = lambda t: t.data_ptr() if pos else None
        check(lib().b200_token_jvp(self._h, xin.data_ptr(), ptr(kc), ptr(vc), pos, self.packed.data_ptr(),
                                   dxin.data_ptr(), packed_dw.data_ptr(), ptr(dkc), ptr(dvc), hidden.data_ptr(),
                                   d_hidden.data_ptr(), ws.data_ptr(), ws.numel(), _stream()))
        return hidden, d_hidden

    def token_vjp(self, x: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, d_hidden: torch.Tensor):
        """Reverse mode of the reference's own call ``forward(x, weights, key_cache, value_cache) -> hidden`` with
        respect to all of its inputs.  ``x`` fp32 [d]; caches [L, pos, d]; ``d_hidden`` fp32 [d].  Returns
        ``(hidden, dx, packed_grads, d_key_cache, d_value_cache)``; ``unpack_grads`` turns the packed gradients into
        the per-leaf dict (``wcls`` and the embedding come out exactly zero: the result does not depend on them)."""
        if not self.with_transposed:
            raise B200Error(1, "token_vjp needs weights packed with with_transposed=True")
        L, d = self.config["n_layers"], self.config["dim"]
        pos = int(key_cache.shape[1])
        if tuple(key_cache.shape) != (L, pos, d) or tuple(value_cache.shape) != (L, pos, d):
            raise B200Error(2, f"caches must be [{L}, pos, {d}], got {tuple(key_cache.shape)} and {tuple(value_cache.shape)}")
        dev = self.device
        xin = x.to(dev, torch.float32).reshape(d).contiguous()
        dh = d_hidden.to(dev, torch.float32).reshape(d).contiguous()
        kc = key_cache.to(dev, self.dtype).contiguous()
        vc = value_cache.to(dev, self.dtype).contiguous()
        hidden = torch.empty(d, dtype=torch.float32, device=dev)
        dx = torch.empty(d, dtype=torch.float32, device=dev)
        dkc = torch.zeros(L, pos, d, dtype=torch.float32, device=dev)
        dvc = torch.zeros(L, pos, d, dtype=torch.float32, device=dev)
        grads = torch.empty(self.grad_bytes() // 4, dtype=torch.float32, device=dev)
        need = self._bytes(lib().b200_token_vjp_workspace_bytes, pos)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        check(lib().b200_token_vjp(self._h, xin.data_ptr(), kc.data_ptr() if pos else None,
                                   vc.data_ptr() if pos else None, pos, self.packed.data_ptr(), dh.data_ptr(),
                                   hidden.data_ptr(), dx.data_ptr(), grads.data_ptr(),
                                   dkc.data_ptr() if pos else None, dvc.data_ptr() if pos else None, ws.data_ptr(),
                                   ws.numel(), _stream()))
        return hidden, dx, grads, dkc, dvc

    # ---- decode ----------------------------------------------------------
    def new_kv_pages(self, n_pages: int, page_size: int) -> torch.Tensor:
        L = self.config["n_layers"]
        hs = self.config["dim"] // self.config["n_heads"]
        return torch.zeros(L, 2, n_pages, self.d_local // hs, page_size, hs, dtype=self.dtype, device=self.device)

    def decode_step(self, pos: int, kv_pages: torch.Tensor, page_table: torch.Tensor, *,
                    tokens: Optional[torch.Tensor] = None, x: Optional[torch.Tensor] = None,
                    want_hidden: bool = False, want_logits: bool = True,
                    logits: Optional[torch.Tensor] = None):
        B = (tokens if tokens is not None else x).shape[0]
        n_pages, page_size = kv_pages.shape[2], kv_pages.shape[4]
        hidden = torch.empty(B, self.config["dim"], dtype=torch.float32, device=self.device) if want_hidden else None
        if want_logits and logits is None:
            logits = torch.empty(B, self.vocab_local, dtype=torch.float32, device=self.device)
        ws = self.workspace(3, B, pos + 1)
        check(lib().b200_decode_step(self._h, _ptr(tokens), _ptr(x), B, pos, self.packed.data_ptr(),
                                     kv_pages.data_ptr(), page_table.data_ptr(), n_pages, page_size,
                                     page_table.shape[1], _ptr(hidden), _ptr(logits) if want_logits else None,
                                     ws.data_ptr(), ws.numel(), _stream()))
        return hidden, (logits if want_logits else None)

    def generate(self, prompt: torch.Tensor, n_new: int, *, page_size: int = 64,
                 kv_pages: Optional[torch.Tensor] = None, allocator: Optional["PageAllocator"] = None) -> torch.Tensor:
        """Greedy decoding: prefill the int32 prompts [B, S0], then ``n_new`` decode steps whose next token is the
        on-device argmax of the step's logits (no logits leave the GPU).  KV rows live in pages taken from
        ``allocator`` (a pool of ``kv_pages``; both are created when absent) and are returned to it at the end.
        Returns int32 [B, S0 + n_new].  One GPU (the vocabulary is not sharded)."""
        if self.tp_size != 1:
            raise B200Error(10, "generate needs the whole vocabulary on one GPU")
        B, S0 = prompt.shape
        total = S0 + n_new
        if total > self.config["seq_len"]:
            raise B200Error(2, f"{total} positions exceed the plan's seq_len={self.config['seq_len']}")
        per_seq = (total + page_size - 1) // page_size
        if kv_pages is None:
            kv_pages = self.new_kv_pages(B * per_seq, page_size)
        if allocator is None:
            allocator = PageAllocator(kv_pages.shape[2])
        owned = []
        try:
            for _ in range(B):
                owned.append(allocator.alloc(per_seq))
            table = torch.tensor(owned, dtype=torch.int32, device=self.device)
            # prefill: logits of every prompt position and the rotated K / V rows, scattered into the pages
            L, H = self.config["n_layers"], self.config["n_heads"]
            hs = self.config["dim"] // H
            kv_flat = torch.empty(L, 2, B, S0, H * hs, dtype=self.dtype, device=self.device)
            logits = self.forward(prompt, kv_out=kv_flat)
            pos = torch.arange(S0, device=self.device)
            pg = table.long()[:, pos // page_size].reshape(-1)            # [B*S0] page of every (sequence, position)
            off = (pos % page_size).repeat(B)
            # advanced indices on the page and row dimensions come first in the indexed view: [B*S0, L, 2, H, hs]
            kv_pages[:, :, pg, :, off, :] = kv_flat.view(L, 2, B * S0, H, hs).permute(2, 0, 1, 3, 4)
            out = torch.empty(B, total, dtype=torch.int32, device=self.device)
            out[:, :S0] = prompt
            cur = argmax(logits[:, -1, :])
            step_logits = torch.empty(B, self.vocab_local, dtype=torch.float32, device=self.device)
            for i in range(n_new):
                out[:, S0 + i] = cur
                if i + 1 == n_new:
                    break
                self.decode_step(S0 + i, kv_pages, table, tokens=cur, logits=step_logits)
                cur = argmax(step_logits)
            return out
        finally:
            for pages in owned:
                allocator.free(pages)
