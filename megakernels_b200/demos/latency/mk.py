"""Bind latency ``Globals`` to the megakernel call.

Reference: megakernels/demos/latency/mk.py:8-54 (argument order and the
``(l b) t h d`` view of the KV cache).
"""

from __future__ import annotations

import torch

from megakernels_b200.demos.latency.instructions import Globals
from megakernels_b200.mk import MK_Interpreter


def interpret_with_mk(globs: Globals, mk_func, stream=None, **kwargs):
    L, B, T, Hkv, D = globs.k_cache.shape
    k4 = globs.k_cache.view(L * B, T, Hkv, D)
    v4 = globs.v_cache.view(L * B, T, Hkv, D)
    return mk_func(
        # vm state
        globs.barriers,
        globs.instructions,
        globs.timings,
        # weights
        globs.qkv_proj_weights,
        globs.attn_ln_weights,
        globs.o_proj_weights,
        globs.mlp_ln_weights,
        globs.up_proj_weights,
        globs.gate_proj_weights,
        globs.down_proj_weights,
        globs.lm_head_norm_weights.data,
        globs.lm_head_weights.data,
        k4,
        v4,
        # rope
        globs.rope_cos,
        globs.rope_sin,
        # activations
        globs.hidden_states,
        globs.post_ln_rope_q,
        globs.attn_out,
        globs.attn_lse_intermediates,
        globs.attn_out_intermediates,
        globs.silu_out,
        globs.logits,
        # scalars
        globs.pos_id,
        globs.attn_scale,
        globs.rms_norm_eps,
        2 if globs.merge_in_last_partial else globs.skip_attn_reduction,
        stream=stream if stream is not None else torch.cuda.current_stream(),
        matvec_reduction_size=globs.matvec_reduction_size,
        residual_scale=globs.residual_scale,
        pos_id_device=globs.pos_id_device,
        tp=globs.tp,
        argmax_out=globs.argmax_out,
        residual_acc=globs.residual_acc,
        upgate_instructions_per_layer=globs.upgate_instructions_per_layer,
        batch=globs.batch_size,
        pos_ids=globs.pos_ids,
        normed_states=globs.normed_states,
        **kwargs,
    )


class LatencyMK_Interpreter(MK_Interpreter):
    def interpret(self, globs: Globals, **kwargs):
        return interpret_with_mk(globs, self.mk_func, **kwargs)
