"""Importable ``mk_llama`` module: a ctypes shim over ``libmkb200.so``.

The reference loads its compiled kernel with ``sys.path.append(mk_dir); from
mk_llama import mk_llama`` (megakernels/mk.py:5-9) and calls it with 23 tensors,
4 scalars and ``stream=`` (megakernels/demos/latency/mk.py:15-49).  This module
offers the same callable.  It only marshals pointers and sizes into the C
struct of ``include/mkb200.h``; all work happens in the CUDA library, and a
missing library is an ImportError, never a fallback.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libmkb200.so"

MKB_ABI_VERSION = 4
MKB_MAX_TP = 8
MKB_TP_MAX_CHUNKS = 32
MKB_PEER_HANDLE_BYTES = 64
MKB_STATUS_WORDS = 16
MKB_FLAG_RECORD_TIMINGS = 1

ERROR_NAMES = {
    0: "MKB_OK",
    1: "MKB_ERR_INVALID_ARGUMENT",
    2: "MKB_ERR_CUDA",
    3: "MKB_ERR_DEVICE_TIMEOUT",
    4: "MKB_ERR_BAD_OPCODE",
    5: "MKB_ERR_UNSUPPORTED",
}


class MkbTensorParallel(ctypes.Structure):
    _fields_ = [
        ("size", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("num_chunks", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("hidden_ll_peers", ctypes.c_void_p * MKB_MAX_TP),
        ("recv_peers", ctypes.c_void_p * MKB_MAX_TP),
        ("partial", ctypes.c_void_p),
        ("epoch_device", ctypes.c_void_p),
    ]


class MkbGlobals(ctypes.Structure):
    _fields_ = [
        ("abi_version", ctypes.c_uint32),
        ("struct_bytes", ctypes.c_uint32),
        ("barriers", ctypes.c_void_p),
        ("instructions", ctypes.c_void_p),
        ("timings", ctypes.c_void_p),
        ("num_sms", ctypes.c_int32),
        ("queue_len", ctypes.c_int32),
        ("barrier_ops", ctypes.c_int32),
        ("barrier_width", ctypes.c_int32),
        ("qkv_weights", ctypes.c_void_p),
        ("attn_ln_weights", ctypes.c_void_p),
        ("o_proj_weights", ctypes.c_void_p),
        ("mlp_ln_weights", ctypes.c_void_p),
        ("up_proj_weights", ctypes.c_void_p),
        ("gate_proj_weights", ctypes.c_void_p),
        ("down_proj_weights", ctypes.c_void_p),
        ("lm_head_norm_weights", ctypes.c_void_p),
        ("lm_head_weights", ctypes.c_void_p),
        ("k_cache", ctypes.c_void_p),
        ("v_cache", ctypes.c_void_p),
        ("rope_cos", ctypes.c_void_p),
        ("rope_sin", ctypes.c_void_p),
        ("hidden_states", ctypes.c_void_p),
        ("post_ln_rope_q", ctypes.c_void_p),
        ("attn_out", ctypes.c_void_p),
        ("attn_lse_intermediates", ctypes.c_void_p),
        ("attn_out_intermediates", ctypes.c_void_p),
        ("silu_out", ctypes.c_void_p),
        ("logits", ctypes.c_void_p),
        ("num_layers", ctypes.c_int32),
        ("hidden_size", ctypes.c_int32),
        ("intermediate_size", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("num_attention_heads", ctypes.c_int32),
        ("num_kv_heads", ctypes.c_int32),
        ("vocab_size", ctypes.c_int32),
        ("kv_max_len", ctypes.c_int32),
        ("kv_batch", ctypes.c_int32),
        ("max_partials", ctypes.c_int32),
        ("matvec_reduction_size", ctypes.c_int32),
        ("pos_id", ctypes.c_int32),
        ("attn_scale", ctypes.c_float),
        ("rms_norm_eps", ctypes.c_float),
        ("skip_attn_reduction", ctypes.c_int32),
        ("pos_id_device", ctypes.c_void_p),
        ("residual_scale", ctypes.c_float),
        ("residual_acc", ctypes.c_void_p),
        ("upgate_instructions_per_layer", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("pos_ids", ctypes.c_int32 * 8),
        ("normed_states", ctypes.c_void_p),
        ("tp", MkbTensorParallel),
        ("argmax_out", ctypes.c_void_p),
        ("flags", ctypes.c_uint32),
        ("wait_timeout_ms", ctypes.c_uint32),
        ("status", ctypes.c_void_p),
    ]


class MkbStatus(ctypes.Structure):
    _fields_ = [
        ("code", ctypes.c_int32),
        ("sm", ctypes.c_int32),
        ("instruction_index", ctypes.c_int32),
        ("opcode", ctypes.c_int32),
        ("role", ctypes.c_int32),
        ("detail", ctypes.c_int32 * 4),
        ("reserved", ctypes.c_int32 * 7),
    ]


class MegakernelError(RuntimeError):
    def __init__(self, code: int, message: str, status: "MkbStatus | None" = None):
        super().__init__(f"{ERROR_NAMES.get(code, code)}: {message}")
        self.code = code
        self.status = status


_lib = None


def load_library() -> ctypes.CDLL:
    """Load ``libmkb200.so``; raise ImportError with build instructions if absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; "
            "g.build()'` (or `make -C megakernels_b200/csrc`). There is no CPU fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.mkb_launch.argtypes = [ctypes.POINTER(MkbGlobals), ctypes.c_void_p]
    lib.mkb_launch.restype = ctypes.c_int
    lib.mkb_launch_no_alloc.argtypes = [ctypes.POINTER(MkbGlobals), ctypes.c_void_p]
    lib.mkb_launch_no_alloc.restype = ctypes.c_int
    lib.mkb_sync_status.argtypes = [
        ctypes.POINTER(MkbGlobals),
        ctypes.c_void_p,
        ctypes.POINTER(MkbStatus),
    ]
    lib.mkb_sync_status.restype = ctypes.c_int
    lib.mkb_sync_status_no_alloc.argtypes = lib.mkb_sync_status.argtypes
    lib.mkb_sync_status_no_alloc.restype = ctypes.c_int
    lib.mkb_peer_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]
    lib.mkb_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    lib.mkb_peer_close.argtypes = [ctypes.c_void_p]
    lib.mkb_peer_free.argtypes = [ctypes.c_void_p]
    for name in ("mkb_peer_alloc", "mkb_peer_open", "mkb_peer_close", "mkb_peer_free"):
        getattr(lib, name).restype = ctypes.c_int
    lib.mkb_last_error.restype = ctypes.c_char_p
    for name in ("mkb_sm_count", "mkb_smem_bytes", "mkb_block_threads", "mkb_abi_version"):
        getattr(lib, name).restype = ctypes.c_int
    if lib.mkb_abi_version() != MKB_ABI_VERSION:
        raise ImportError(
            f"libmkb200.so has ABI {lib.mkb_abi_version()}, this shim expects {MKB_ABI_VERSION}"
        )
    _lib = lib
    return lib


def _check_tensor(name, t, dtype, ndim=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must live on a CUDA device")
    # the launch goes to the current device: a tensor elsewhere would be a wild pointer there
    if t.device.index != torch.cuda.current_device():
        raise ValueError(
            f"{name} lives on cuda:{t.device.index} but the current device is "
            f"cuda:{torch.cuda.current_device()} (wrap the call in torch.cuda.device(...))"
        )
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if ndim is not None and t.ndim != ndim:
        raise ValueError(f"{name} must have {ndim} dimensions, got {tuple(t.shape)}")
    return t.data_ptr()


def pack_globals(
    barriers,
    instructions,
    timings,
    qkv_weights,
    attn_ln_weights,
    o_proj_weights,
    mlp_ln_weights,
    up_proj_weights,
    gate_proj_weights,
    down_proj_weights,
    lm_head_norm_weights,
    lm_head_weights,
    k_cache,
    v_cache,
    rope_cos,
    rope_sin,
    hidden_states,
    post_ln_rope_q,
    attn_out,
    attn_lse_intermediates,
    attn_out_intermediates,
    silu_out,
    logits,
    pos_id,
    attn_scale,
    rms_norm_eps,
    skip_attn_reduction,
    matvec_reduction_size=None,
    wait_timeout_ms=0,
    status=None,
    record_timings=False,
    num_attention_heads=None,
    max_partials=None,
    pos_id_device=None,
    residual_scale=1.0,
    tp=None,
    argmax_out=None,
    residual_acc=None,
    upgate_instructions_per_layer=0,
    batch=1,
    pos_ids=None,
    normed_states=None,
) -> MkbGlobals:
    """Fill the C struct from tensors; every dimension is read off the shapes."""
    bf16, i32, f32 = torch.bfloat16, torch.int32, torch.float32
    g = MkbGlobals()
    g.abi_version = MKB_ABI_VERSION
    g.struct_bytes = ctypes.sizeof(MkbGlobals)
    g.barriers = _check_tensor("barriers", barriers, i32, 3)
    g.instructions = _check_tensor("instructions", instructions, i32, 3)
    g.timings = _check_tensor("timings", timings, i32, 3) if timings is not None else None
    g.num_sms, g.queue_len = instructions.shape[0], instructions.shape[1]
    if instructions.shape[2] != 32:
        raise ValueError("instructions must be [num_sms, queue_len, 32]")
    g.barrier_ops, g.barrier_width = barriers.shape[1], barriers.shape[2]

    g.qkv_weights = _check_tensor("qkv_weights", qkv_weights, bf16, 3)
    g.attn_ln_weights = _check_tensor("attn_ln_weights", attn_ln_weights, bf16, 2)
    g.o_proj_weights = _check_tensor("o_proj_weights", o_proj_weights, bf16, 3)
    g.mlp_ln_weights = _check_tensor("mlp_ln_weights", mlp_ln_weights, bf16, 2)
    g.up_proj_weights = _check_tensor("up_proj_weights", up_proj_weights, bf16, 3)
    g.gate_proj_weights = _check_tensor("gate_proj_weights", gate_proj_weights, bf16, 3)
    g.down_proj_weights = _check_tensor("down_proj_weights", down_proj_weights, bf16, 3)
    g.lm_head_norm_weights = _check_tensor("lm_head_norm_weights", lm_head_norm_weights, bf16, 1)
    g.lm_head_weights = _check_tensor("lm_head_weights", lm_head_weights, bf16, 2)
    g.k_cache = _check_tensor("k_cache", k_cache, bf16, 4)
    g.v_cache = _check_tensor("v_cache", v_cache, bf16, 4)
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    g.rope_cos = _check_tensor("rope_cos", rope_cos, f32, 2)
    g.rope_sin = _check_tensor("rope_sin", rope_sin, f32, 2)
    g.hidden_states = _check_tensor("hidden_states", hidden_states, bf16)
    g.post_ln_rope_q = _check_tensor("post_ln_rope_q", post_ln_rope_q, bf16)
    g.attn_out = _check_tensor("attn_out", attn_out, bf16)
    if attn_lse_intermediates is None and attn_out_intermediates is None:
        # only valid for mk_llama_no_alloc, which supplies its own scratch
        if num_attention_heads is None or max_partials is None:
            raise ValueError("without intermediates, num_attention_heads and max_partials are needed")
        g.attn_lse_intermediates = None
        g.attn_out_intermediates = None
    else:
        g.attn_lse_intermediates = _check_tensor("attn_lse_intermediates", attn_lse_intermediates, f32)
        g.attn_out_intermediates = _check_tensor("attn_out_intermediates", attn_out_intermediates, f32)
        if attn_lse_intermediates.ndim not in (2, 3) or attn_out_intermediates.ndim != attn_lse_intermediates.ndim + 1:
            raise ValueError("attention intermediates must be [(batch,) Hq, P] and [(batch,) Hq, P, D]")
        num_attention_heads = attn_lse_intermediates.shape[-2]
        max_partials = attn_lse_intermediates.shape[-1]
    g.silu_out = _check_tensor("silu_out", silu_out, bf16)
    g.logits = _check_tensor("logits", logits, bf16)

    L, qkv_rows, H = qkv_weights.shape
    LB, T, Hkv, D = k_cache.shape
    Hq = int(num_attention_heads)
    g.num_layers = L
    g.hidden_size = H
    g.intermediate_size = up_proj_weights.shape[1]
    g.head_dim = D
    g.num_attention_heads = Hq
    g.num_kv_heads = Hkv
    g.vocab_size = lm_head_weights.shape[0]
    g.kv_max_len = T
    g.kv_batch = LB // L
    g.max_partials = int(max_partials)
    if qkv_rows != (Hq + 2 * Hkv) * D:
        raise ValueError(
            f"qkv rows {qkv_rows} != (Hq + 2*Hkv)*D = {(Hq + 2 * Hkv) * D}"
        )
    if rope_cos.shape[1] != D or rope_sin.shape != rope_cos.shape:
        raise ValueError("rope tables must be [positions, head_dim]")
    if pos_id_device is not None:
        g.pos_id_device = _check_tensor("pos_id_device", pos_id_device, i32)
        # the kernel bounds a device-side position by the KV length only, so the RoPE
        # tables must cover every position the cache can hold
        if rope_cos.shape[0] < T:
            raise ValueError(
                f"with pos_id_device the rope tables need >= kv_max_len = {T} rows, got {rope_cos.shape[0]}"
            )
    elif rope_cos.shape[0] <= int(pos_id):
        raise ValueError(f"rope tables have {rope_cos.shape[0]} rows, pos_id is {pos_id}")
    if matvec_reduction_size is None:
        for r in (2048, 1024, 512, 256):
            if (Hq * D) % r == 0 and g.intermediate_size % r == 0:
                matvec_reduction_size = r
                break
        else:
            raise ValueError("cannot derive matvec_reduction_size from the shapes")
    g.matvec_reduction_size = int(matvec_reduction_size)
    g.pos_id = int(pos_id)
    g.attn_scale = float(attn_scale)
    g.rms_norm_eps = float(rms_norm_eps)
    # 0: AttentionReduction instructions, 1: one partition writes attn_out, 2: the last partial merges
    g.skip_attn_reduction = 2 if (skip_attn_reduction is not True and skip_attn_reduction == 2) else int(bool(skip_attn_reduction))
    g.residual_scale = float(residual_scale)
    if tp is not None:
        # megakernels_b200.instructions.TensorParallelState with its buffers attached
        if tp.hidden_ptrs is None or tp.partial is None or tp.epoch_device is None:
            raise ValueError("tensor-parallel state has no peer buffers attached (peer.connect)")
        g.tp.size, g.tp.rank, g.tp.num_chunks = tp.size, tp.rank, tp.num_chunks
        for r in range(tp.size):
            g.tp.hidden_ll_peers[r] = tp.hidden_ptrs[r]
            g.tp.recv_peers[r] = tp.recv_ptrs[r]
        g.tp.partial = _check_tensor("tp.partial", tp.partial, f32, 2)
        g.tp.epoch_device = _check_tensor("tp.epoch_device", tp.epoch_device, i32)
    if argmax_out is not None:
        g.argmax_out = _check_tensor("argmax_out", argmax_out, i32)
    batch = int(batch or 1)
    if residual_acc is not None:
        g.residual_acc = _check_tensor("residual_acc", residual_acc, torch.int64)
        if residual_acc.numel() < batch * H:
            raise ValueError(f"residual_acc needs {batch * H} int64 elements, got {residual_acc.numel()}")
    if batch > 1:
        # batched decode: leading batch dimension on the activation tensors
        for name, t, n in (
            ("hidden_states", hidden_states, H), ("post_ln_rope_q", post_ln_rope_q, Hq * D),
            ("attn_out", attn_out, Hq * D), ("silu_out", silu_out, g.intermediate_size),
            ("logits", logits, g.vocab_size),
        ):
            if tuple(t.shape) != (batch, n):
                raise ValueError(f"{name} must be [{batch}, {n}] for a batch of {batch}, got {tuple(t.shape)}")
        g.batch = batch
        g.normed_states = _check_tensor("normed_states", normed_states, bf16, 2)
        if pos_id_device is None:
            if batch > 8:
                raise ValueError("more than 8 sequences need pos_id_device (int32, one position per sequence)")
            if pos_ids is None or len(pos_ids) != batch:
                raise ValueError("a batched launch needs pos_ids (one position per sequence) or pos_id_device")
            for s, pos in enumerate(pos_ids):
                if not 0 <= int(pos) < min(T, rope_cos.shape[0]):
                    raise ValueError(f"pos_ids[{s}] = {pos} outside the KV cache / rope tables")
                g.pos_ids[s] = int(pos)
        elif pos_id_device.numel() < batch:
            raise ValueError("pos_id_device must hold one position per sequence")
        if argmax_out is not None and argmax_out.numel() < batch:
            raise ValueError("argmax_out must hold one token per sequence")
    g.upgate_instructions_per_layer = int(upgate_instructions_per_layer)
    g.flags = MKB_FLAG_RECORD_TIMINGS if record_timings else 0
    if record_timings and timings is None:
        raise ValueError("record_timings needs the timings tensor")
    g.wait_timeout_ms = int(wait_timeout_ms)
    g.status = _check_tensor("status", status, i32) if status is not None else None
    return g


_residual_accs: dict = {}


def _own_residual_acc(hidden_states, stream):
    """Accumulator for callers of the bare reference signature, zeroed on the launch stream."""
    key = (hidden_states.device.index, hidden_states.data_ptr(), hidden_states.numel())
    acc = _residual_accs.get(key)
    if acc is None:
        if len(_residual_accs) >= 16:
            _residual_accs.clear()
        acc = _residual_accs[key] = torch.zeros(
            hidden_states.numel(), dtype=torch.int64, device=hidden_states.device
        )
    ctx = torch.cuda.stream(stream) if isinstance(stream, torch.cuda.Stream) else None
    if ctx is None:
        acc.zero_()
    else:
        with ctx:
            acc.zero_()
    return acc


def _stream_handle(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    if isinstance(stream, int):
        return stream
    return int(stream.cuda_stream)


def mk_llama(
    *args,
    stream=None,
    matvec_reduction_size=None,
    wait_timeout_ms=0,
    status=None,
    record_timings=False,
    pos_id_device=None,
    residual_scale=1.0,
    tp=None,
    argmax_out=None,
    residual_acc=None,
    upgate_instructions_per_layer=0,
    batch=1,
    pos_ids=None,
    normed_states=None,
):
    """Enqueue one decode step; positional arguments as in the reference call.

    ``(barriers, instructions, timings, qkv_w, attn_ln_w, o_w, mlp_ln_w, up_w,
    gate_w, down_w, lm_head_norm_w, lm_head_w, k_cache4d, v_cache4d, rope_cos,
    rope_sin, hidden_states, post_ln_rope_q, attn_out, attn_lse_intermediates,
    attn_out_intermediates, silu_out, logits, pos_id, attn_scale, rms_norm_eps,
    skip_attn_reduction, stream=...)``.  Asynchronous; raises
    ``MegakernelError`` when host-side validation rejects the arguments.

    ``residual_acc`` (int64 ``[H]``, zero before the launch) is where the kernel sums the
    o-proj / down-proj outputs; a caller that passes only the reference's 27 arguments gets
    one per ``hidden_states`` buffer from this module, cleared on the launch stream before
    every call (one small memset more than a caller who resets it with the barriers).
    """
    if len(args) != 27:
        raise TypeError(f"mk_llama expects 27 positional arguments, got {len(args)}")
    lib = load_library()
    if residual_acc is None and tp is None:
        residual_acc = _own_residual_acc(args[16], stream)
    g = pack_globals(
        *args,
        matvec_reduction_size=matvec_reduction_size,
        wait_timeout_ms=wait_timeout_ms,
        status=status,
        record_timings=record_timings,
        pos_id_device=pos_id_device,
        residual_scale=residual_scale,
        tp=tp,
        argmax_out=argmax_out,
        residual_acc=residual_acc,
        upgate_instructions_per_layer=upgate_instructions_per_layer,
        batch=batch,
        pos_ids=pos_ids,
        normed_states=normed_states,
    )
    rc = lib.mkb_launch(ctypes.byref(g), ctypes.c_void_p(_stream_handle(stream)))
    if rc != 0:
        raise MegakernelError(rc, lib.mkb_last_error().decode())
    return g


def peer_alloc(nbytes: int) -> tuple[int, bytes]:
    """Zero-filled peer-visible device memory on the current device: (address, 64-byte handle)."""
    lib = load_library()
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(MKB_PEER_HANDLE_BYTES)
    rc = lib.mkb_peer_alloc(nbytes, ctypes.byref(ptr), handle)
    if rc != 0:
        raise MegakernelError(rc, lib.mkb_last_error().decode())
    return int(ptr.value), handle.raw


def peer_open(handle: bytes) -> int:
    """Map another process's peer_alloc block into this process; returns the local address."""
    lib = load_library()
    ptr = ctypes.c_void_p()
    rc = lib.mkb_peer_open(ctypes.create_string_buffer(handle, MKB_PEER_HANDLE_BYTES), ctypes.byref(ptr))
    if rc != 0:
        raise MegakernelError(rc, lib.mkb_last_error().decode())
    return int(ptr.value)


def peer_close(ptr: int) -> None:
    load_library().mkb_peer_close(ctypes.c_void_p(ptr))


def peer_free(ptr: int) -> None:
    load_library().mkb_peer_free(ctypes.c_void_p(ptr))


def sync_status(g: MkbGlobals, stream=None, no_alloc: bool = False) -> MkbStatus:
    """Synchronise the stream and return the device status; raise on device errors.

    ``no_alloc`` selects ``mkb_sync_status_no_alloc``, the read-back that belongs to
    :func:`mk_llama_no_alloc` (it finds the record in the library's static array when the
    caller passed no ``status`` tensor, and never allocates).
    """
    lib = load_library()
    st = MkbStatus()
    fn = lib.mkb_sync_status_no_alloc if no_alloc else lib.mkb_sync_status
    rc = fn(ctypes.byref(g), ctypes.c_void_p(_stream_handle(stream)), ctypes.byref(st))
    if rc != 0:
        msg = lib.mkb_last_error().decode()
        raise MegakernelError(rc, msg, st)
    return st


def mk_llama_no_alloc(
    *args,
    stream=None,
    matvec_reduction_size=None,
    wait_timeout_ms=0,
    status=None,
    num_attention_heads=None,
    max_partials=None,
    upgate_instructions_per_layer=0,
):
    """One decode step through ``mkb_launch_no_alloc``: nothing is allocated by the call.

    Same 27 positional arguments as :func:`mk_llama`; pass ``None`` for the two
    attention intermediates together with ``num_attention_heads`` and
    ``max_partials`` - the library keeps that scratch (and, unless ``status`` is
    given, its error record) in a static device array, for callers whose device
    memory is fully planned and who therefore cannot let a library call cudaMalloc.
    The residual accumulators live in the same array and are cleared by the call.
    The array is shared by all calls: do not overlap two of them on the GPU.
    """
    if len(args) != 27:
        raise TypeError(f"mk_llama_no_alloc expects 27 positional arguments, got {len(args)}")
    lib = load_library()
    g = pack_globals(
        *args,
        matvec_reduction_size=matvec_reduction_size,
        wait_timeout_ms=wait_timeout_ms,
        status=status,
        num_attention_heads=num_attention_heads,
        max_partials=max_partials,
        upgate_instructions_per_layer=upgate_instructions_per_layer,
    )
    rc = lib.mkb_launch_no_alloc(ctypes.byref(g), ctypes.c_void_p(_stream_handle(stream)))
    if rc != 0:
        raise MegakernelError(rc, lib.mkb_last_error().decode())
    return g
