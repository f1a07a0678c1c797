"""Generic instruction-set base: kernel globals and instruction encoding.

Reference: megakernels/instructions.py.  ``BaseGlobals`` is the argument set
of the megakernel (:10-69); ``Instruction.serialize`` defines the int32 word
layout the device decodes (:83-119); ``NoOp`` is opcode 0 (:122-126).
"""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any

from torch import Tensor

from megakernels_b200.model_types import DeviceType
from megakernels_b200.utils import get_sm_count


TP_MAX_RANKS = 8  # MKB_MAX_TP
TP_MAX_CHUNKS = 32  # MKB_TP_MAX_CHUNKS


@dataclass
class TensorParallelState:
    """Host mirror of ``MkbTensorParallel`` (include/mkb200.h): the in-kernel all-reduce.

    No counterpart in the reference, whose kernel is single-GPU.  ``size``,
    ``rank`` and ``num_chunks`` are known when the schedule is built (the
    builder emits one ``TP_AllReduce`` instruction per chunk after every o-proj
    and down-proj group); the buffers are attached later by whoever owns the
    exchange: ``megakernels_b200.peer.connect`` for GPUs (peer-mapped memory),
    the CPU checker for its own emulation (``exchange`` callback).
    """

    size: int
    rank: int
    num_chunks: int
    epoch: int = 0  # launches completed so far; mirrors ``epoch_device``
    partial: Tensor | None = None  # fp32 [max slices, H], local
    recv: Tensor | None = None  # int32 [size, H/2, 4] = {f32, tag, f32, tag}, written by peers
    hidden_tagged: Tensor | None = None  # int32 [H/2, 2] = {bf16x2, tag}: the running residual stream
    counters: Tensor | None = None  # CPU checker only: int32 [L, 2, 1 + TP_MAX_CHUNKS] arrival counts
    epoch_device: Tensor | None = None  # int32 [1]
    hidden_ptrs: list[int] | None = None  # device address of the tagged residual buffer on every rank
    recv_ptrs: list[int] | None = None
    exchange: Any = None  # CPU checker only: fp32 tensor -> sum over ranks

    def __post_init__(self):
        assert 1 < self.size <= TP_MAX_RANKS and 0 <= self.rank < self.size
        assert self.num_chunks % self.size == 0 and self.num_chunks <= TP_MAX_CHUNKS

    def owner(self, chunk: int) -> int:
        return chunk % self.size


@dataclass
class BaseGlobals:
    # model parameters, stacked over layers
    qkv_proj_weights: Tensor
    attn_ln_weights: Tensor
    o_proj_weights: Tensor
    mlp_ln_weights: Tensor
    up_proj_weights: Tensor
    gate_proj_weights: Tensor
    down_proj_weights: Tensor
    lm_head_norm_weights: Tensor
    lm_head_weights: Tensor
    k_cache: Tensor
    v_cache: Tensor

    # shared by all layers
    rope_cos: Tensor
    rope_sin: Tensor

    # model constants (per-rank values under tensor parallelism)
    num_hidden_layers: int
    num_attention_heads: int
    num_kv_heads: int
    head_dim: int
    hidden_size: int
    intermediate_size: int
    vocab_size: int

    attn_scale: float
    rms_norm_eps: float
    device: DeviceType

    hidden_states: Tensor
    barriers: Tensor

    pos_id: int

    def __post_init__(self):
        self.instructions: Tensor | None = None
        self.timings: Tensor | None = None
        # extensions without a counterpart in the reference globals
        self.residual_scale: float = 1.0  # tensor-parallel degree (see generators.TP_MK_Generator)
        self.pos_id_device: Tensor | None = None  # int32[1]; overrides pos_id when set
        self.tp: TensorParallelState | None = None  # in-kernel tensor-parallel all-reduce
        self.argmax_out: Tensor | None = None  # int32[1]: the kernel's own argmax over the logits
        # split-KV schedules without AttentionReduction instructions: the last partial of a KV head
        # to arrive merges the partial rows itself (launched as skip_attn_reduction = 2)
        self.merge_in_last_partial: bool = False
        # int64 [H]: the token's o-proj / down-proj outputs summed in Q31.32 fixed point by the
        # kernel (integer atomics: the same bits whatever order the SMs arrive in).  The kernel
        # never writes ``hidden_states``; the residual stream is ``residual_stream()``.
        self.residual_acc: Tensor | None = None
        # one int32 buffer behind ``barriers`` and ``residual_acc``, so that a single fill
        # resets both before a launch
        self.vm_state: Tensor | None = None
        # RMS + up/gate instructions per layer of the schedule (0: unknown); the down-proj
        # waits for that many residual-stream reads before it adds to the accumulators
        self.upgate_instructions_per_layer: int = 0
        # batched decode: sequences per launch, their positions (host list, or a device int32
        # tensor in ``pos_id_device``), and the buffer RMS_Norm instructions write
        self.batch_size: int = 1
        self.pos_ids: list[int] | None = None
        self.normed_states: Tensor | None = None

    def residual_stream(self) -> Tensor:
        """The residual stream after a launch as fp32 ``[H]``: embedding + accumulated outputs.

        The CPU checker follows the reference and adds into ``hidden_states`` itself, so its
        accumulators stay zero and this is just ``hidden_states`` there.
        """
        h = self.hidden_states.float()
        if self.residual_acc is not None:
            h = (h.double() + self.residual_acc.double() * 2.0**-32).float()
        return h

    def sm_count(self) -> int:
        return get_sm_count(self.device)

    def num_total_heads(self) -> int:
        return self.num_attention_heads + self.num_kv_heads * 2

    def diff(self, other: "BaseGlobals", skip_kv_cache: bool = False, verbose: bool = True):
        """Compare every non-weight tensor of two globals.

        Reference: megakernels/instructions.py:54-66.  Returns
        ``{name: (max_abs_diff, mean_rel_diff)}`` in addition to printing.
        """
        out = {}
        for f in fields(self):
            a, b = getattr(self, f.name), getattr(other, f.name)
            if (
                not isinstance(a, Tensor)
                or "weights" in f.name
                or f.name in ("rope_cos", "rope_sin")
                or (skip_kv_cache and "cache" in f.name)
            ):
                continue
            _, adiff, rdiff = diff_tensors(a, b, f.name, verbose=verbose)
            out[f.name] = (float(adiff.max()), float(rdiff.mean()))
        return out


def diff_tensors(a: Tensor, b: Tensor, name: str, verbose: bool = True):
    """Reference: megakernels/instructions.py:72-80."""
    a = a.float().cpu()
    b = b.float().cpu()
    diff = a - b
    adiff = diff.abs()
    rdiff = 2 * adiff / (a.abs() + b.abs() + 1e-6)
    if verbose:
        print(f"{name}: max adiff: {adiff.max()}, mean rdiff: {rdiff.mean()}")
    return diff, adiff, rdiff


@dataclass
class Instruction:
    @classmethod
    def opcode(cls) -> int:
        raise NotImplementedError

    @classmethod
    def prev_opcode(cls) -> int:
        raise NotImplementedError

    @classmethod
    def tags(cls) -> dict[str, Any]:
        return {}

    def cost(self, globs) -> float:
        return 0.0

    def serialize(self) -> list[int]:
        """Word layout: opcode, then the dataclass fields in declaration order.

        Ints (and bools) take one word, ``None`` becomes 0, tuples and lists
        are length-prefixed, and a field named ``global_idx`` is skipped
        (reference: megakernels/instructions.py:97-119).  ``batch_idx`` (always the
        last field, no counterpart in the reference) is only written when non-zero.
        """
        words = [self.opcode()]
        for f in fields(self):
            if f.name == "global_idx":
                continue
            v = getattr(self, f.name)
            if f.name == "batch_idx" and v == 0:
                # trailing sequence index of a batched launch: absent for sequence 0, so that a
                # single-sequence stream is word for word the reference's (the padding is zero)
                continue
            if isinstance(v, int):
                words.append(int(v))
            elif isinstance(v, (tuple, list)):
                words.append(len(v))
                words.extend(int(x) for x in v)
            elif v is None:
                words.append(0)
            else:
                raise ValueError(f"Unsupported field type: {v!r}")
        return words


@dataclass
class NoOp(Instruction):
    @classmethod
    def opcode(cls) -> int:
        return 0
