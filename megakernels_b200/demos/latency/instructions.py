"""The seven-opcode latency instruction set and its kernel globals.

Reference: megakernels/demos/latency/instructions.py.  Word layouts (after
``Instruction.serialize``) as the device decodes them:

====  ==============================  ==========================================
 op   class                           words
====  ==============================  ==========================================
 1    LayerNorm_QKV_MatVecRopeAppend  [1, layer, start_blk, end_blk]
 2    PartialAttention                [2, layer, kv_head, num_partials, partial]
 3    AttentionReduction              [3, layer, head_start, num_partials,
                                       is_terminal, n, idx_0..idx_{n-1}, out_idx]
 4    O_ProjResidual                  [4, layer, start_blk, end_blk, red_blk]
 5    LayerNormDoubleMatVecSiLU       [5, layer, n, blk_0..blk_{n-1}]
 6    DownProjResidual                [6, layer, start_blk, end_blk, red_blk]
 7    RMS_LM_Head                     [7, start_blk, end_blk]
 8    TP_AllReduce                    [8, layer, which, chunk, num_chunks]
 9    RMS_Norm                        [9, layer, which, sequence]
====  ==============================  ==========================================

Batched decode (``Globals.batch_size`` > 1, no counterpart in the reference's latency
kernel): opcode 2 carries the sequence as a sixth word, opcode 3 as the word after
``out_idx`` (both 0 for a single sequence, where the padded words equal the reference's),
and opcode 9 normalises one sequence's residual stream for all SMs (``which`` 0: attention
norm, 1: MLP norm, 2: final norm); opcodes 1, 5 and 7 then wait for one arrival per sequence
in barrier row 9 instead of normalising themselves.

Opcode 8 has no counterpart in the reference: it is one chunk of the in-kernel
tensor-parallel all-reduce of the residual stream (``which`` 0: after the
o-proj, 1: after the down-proj), only scheduled when ``globs.tp`` is set.

A block is 16 output rows.  ``red_blk`` selects the input-column slice
``[red_blk * matvec_reduction_size, (red_blk + 1) * matvec_reduction_size)``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from torch import Tensor

from megakernels_b200.instructions import BaseGlobals, Instruction


@dataclass
class Globals(BaseGlobals):
    # activation buffers (reference: latency/instructions.py:9-29)
    post_ln_rope_q: Tensor
    attn_out: Tensor
    attn_lse_intermediates: Tensor
    attn_out_intermediates: Tensor
    silu_out: Tensor
    logits: Tensor

    skip_attn_reduction: bool

    # block size constants
    up_gate_proj_block_size: int
    down_proj_block_size: int
    o_proj_block_size: int
    lm_head_block_size: int
    matvec_reduction_size: int
    qkv_block_size: int
    attn_kv_block_size: int
    attn_reduction_size: int

    def o_proj_in_features(self) -> int:
        return self.num_attention_heads * self.head_dim

    def num_o_proj_col_splits(self) -> int:
        return self.o_proj_in_features() // self.matvec_reduction_size

    def num_down_proj_col_splits(self) -> int:
        return self.intermediate_size // self.matvec_reduction_size

    def barrier_thresholds(self) -> dict[str, int]:
        """Counter values each opcode waits for, derived from the shapes.

        At the Llama-3.2-1B shape these are the constants the reference
        hard-codes: 512 (down-proj blocks, rms_matvec_rope_append.cu:49-60),
        4 (blocks per head, attention_partial.cu:314-326), 32 (heads,
        matvec_adds.cu:187-192), 128 (o-proj blocks, upgate.cu:32-40) and
        128 (up/gate blocks per reduction slice, matvec_adds.cu:181-186).
        """
        hidden_blocks = self.hidden_size // self.down_proj_block_size
        return {
            "qkv_waits_downproj": hidden_blocks * self.num_down_proj_col_splits(),
            "attn_waits_qkv_per_head": self.head_dim // self.qkv_block_size,
            "oproj_waits_attn": self.num_attention_heads,
            "upgate_waits_oproj": (self.hidden_size // self.o_proj_block_size)
            * self.num_o_proj_col_splits(),
            "downproj_waits_upgate": self.matvec_reduction_size // self.up_gate_proj_block_size,
        }


@dataclass
class LayerNorm_QKV_MatVecRopeAppend(Instruction):
    """RMSNorm + QKV matvec + RoPE on q/k + append k/v to the KV cache."""

    layer_idx: int
    start_output_block_idx: int
    end_output_block_idx: int

    @classmethod
    def opcode(cls) -> int:
        return 1

    @classmethod
    def prev_opcode(cls) -> int:
        return DownProjResidual.opcode()

    def block_indices(self):
        return list(range(self.start_output_block_idx, self.end_output_block_idx))

    def cost(self, globs: Globals):
        n = self.end_output_block_idx - self.start_output_block_idx
        return n * globs.qkv_block_size * globs.hidden_size


@dataclass
class PartialAttention(Instruction):
    """GQA decode attention of one KV head over one slice of the sequence."""

    layer_idx: int
    kv_head_idx: int
    num_partials: int
    partial_idx: int
    batch_idx: int = 0

    @classmethod
    def opcode(cls) -> int:
        return 2

    @classmethod
    def prev_opcode(cls) -> int:
        return LayerNorm_QKV_MatVecRopeAppend.opcode()

    def cost(self, globs: Globals):
        seq_len = globs.pos_id + 1
        return (seq_len / self.num_partials) * globs.head_dim * 2


@dataclass
class AttentionReduction(Instruction):
    """Merge ``reduction_list`` partial (O, LSE) pairs of 4 consecutive Q heads."""

    layer_idx: int
    head_start_idx: int
    num_partials: int
    is_terminal: bool
    reduction_list: list[int]
    output_partial_idx: Optional[int] = None
    batch_idx: int = 0

    @classmethod
    def opcode(cls) -> int:
        return 3

    @classmethod
    def prev_opcode(cls) -> int:
        return PartialAttention.opcode()

    def cost(self, globs: Globals):
        return len(self.reduction_list) * globs.attn_reduction_size * (globs.head_dim + 1) * 2


@dataclass
class MatVecAdd(Instruction):
    layer_idx: int
    start_block_idx: int
    end_block_idx: int
    reduction_block_idx: int


@dataclass
class O_ProjResidual(MatVecAdd):
    @classmethod
    def opcode(cls) -> int:
        return 4

    @classmethod
    def prev_opcode(cls) -> int:
        return AttentionReduction.opcode()

    def cost(self, globs: Globals):
        n = self.end_block_idx - self.start_block_idx
        return n * globs.o_proj_block_size * min(
            globs.matvec_reduction_size, globs.o_proj_in_features()
        )


@dataclass
class LayerNormDoubleMatVecSiLU(Instruction):
    """RMSNorm + up and gate matvecs + SiLU(gate) * up."""

    layer_idx: int
    block_idxs: list[int]

    @classmethod
    def opcode(cls) -> int:
        return 5

    @classmethod
    def prev_opcode(cls) -> int:
        return O_ProjResidual.opcode()

    def cost(self, globs: Globals):
        return len(self.block_idxs) * globs.up_gate_proj_block_size * globs.hidden_size * 2


@dataclass
class DownProjResidual(MatVecAdd):
    @classmethod
    def opcode(cls) -> int:
        return 6

    @classmethod
    def prev_opcode(cls) -> int:
        return LayerNormDoubleMatVecSiLU.opcode()

    def cost(self, globs: Globals):
        n = self.end_block_idx - self.start_block_idx
        return n * globs.down_proj_block_size * globs.matvec_reduction_size


@dataclass
class TP_AllReduce(Instruction):
    """One chunk of the all-reduce of the row-split projections' partial sums.

    Sums this rank's column slices for elements ``[chunk * H / num_chunks, ...)``,
    sends them to rank ``chunk % tp.size``; that rank adds all ranks' sums to the
    residual stream in fp32, rounds to bf16 once and writes the chunk into every
    rank's ``hidden_states``.
    """

    layer_idx: int
    which: int  # 0: after o-proj, 1: after down-proj
    chunk_idx: int
    num_chunks: int

    @classmethod
    def opcode(cls) -> int:
        return 8

    @classmethod
    def prev_opcode(cls) -> int:
        raise NotImplementedError("depends on `which`")

    def producer_opcode(self) -> int:
        return O_ProjResidual.opcode() if self.which == 0 else DownProjResidual.opcode()

    def cost(self, globs: Globals):
        return globs.hidden_size // self.num_chunks * 64


@dataclass
class RMS_Norm(Instruction):
    """Batched decode only: RMSNorm of one sequence's residual stream into ``normed_states``."""

    layer_idx: int
    which: int  # 0: attention norm of the layer, 1: its MLP norm, 2: the final norm
    batch_idx: int

    @classmethod
    def opcode(cls) -> int:
        return 9

    def cost(self, globs: Globals):
        return globs.hidden_size * 8


@dataclass
class RMS_LM_Head(Instruction):
    start_output_block_idx: int
    end_output_block_idx: int

    @classmethod
    def opcode(cls) -> int:
        return 7

    @classmethod
    def prev_opcode(cls) -> int:
        return DownProjResidual.opcode()

    def cost(self, globs: Globals):
        n = self.end_output_block_idx - self.start_output_block_idx
        return n * globs.lm_head_block_size * globs.hidden_size
