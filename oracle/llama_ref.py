"""CPU checker: the reference's plain-torch Llama decode step, restated.

TEST INFRASTRUCTURE, NOT A PRODUCT PATH.  Only tests, the smoke check and the
benchmark's CPU-baseline leg may import this module.

Restates the torch path of the reference (``PyTorchGenerator`` ->
``LlamaForCausalLM.forward``, megakernels/generators.py:61-92,
megakernels/llama.py:232-296, 328-348, 384-403, 529-550) for one decoded token
over stacked weights: RMSNorm in fp32 rounded to the storage dtype before the
weight multiply, ``F.linear`` projections, interleaved RoPE evaluated in fp32,
KV append at ``pos``, ``scaled_dot_product_attention`` with ``enable_gqa`` over
``cache[:pos+1]``, residual adds in the storage dtype, SiLU-gated MLP, final
norm and LM head.  This path is shape-generic, which the reference's Python VM
is not, so it is the oracle for the 8B / 70B shapes.

Parity status: pinned against outputs of the reference's own torch path run in
the build container (tests/golden/torch_*.pt).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

from oracle.python_vm import rms_norm, rope_interleaved


class TorchReferenceModel:
    """Holds CPU copies of the (unsharded) stacked weights and its own KV cache."""

    def __init__(self, model, kv_len: int | None = None):
        cfg = model.config
        self.cfg = cfg
        sp = model.stacked_params
        cpu = lambda t: t.detach().to("cpu")  # noqa: E731
        self.qkv = cpu(sp.qkv_proj)
        self.o = cpu(sp.o_proj)
        self.up = cpu(sp.up_proj)
        self.gate = cpu(sp.gate_proj)
        self.down = cpu(sp.down_proj)
        self.attn_ln = cpu(sp.attn_ln_weight)
        self.mlp_ln = cpu(sp.mlp_ln_weight)
        self.final_norm = cpu(model.lm_head.input_norm.weight)
        self.head = cpu(model.lm_head.lm_head.weight)
        self.embed = cpu(model.model.embed_tokens.embed_tokens.weight)
        self.rope_cos = cpu(model.model.rope_cos)
        self.rope_sin = cpu(model.model.rope_sin)
        self.eps = cfg.rms_norm_eps
        self.Hq = self.qkv.shape[1] // cfg.head_dim - 2 * model.num_kv_heads()
        self.Hkv = model.num_kv_heads()
        self.D = cfg.head_dim
        T = kv_len or model.kv_len()
        L = cfg.num_hidden_layers
        self.k_cache = torch.zeros(L, 1, T, self.Hkv, self.D, dtype=self.qkv.dtype)
        self.v_cache = torch.zeros_like(self.k_cache)

    def load_kv(self, k_cache: Tensor, v_cache: Tensor):
        self.k_cache = k_cache.detach().to("cpu").clone()
        self.v_cache = v_cache.detach().to("cpu").clone()

    @torch.no_grad()
    def decode_hidden(self, hidden: Tensor, pos: int) -> Tensor:
        """One token through all layers; ``hidden`` is ``[H]`` in storage dtype."""
        h = hidden.reshape(1, 1, -1).clone()
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        cos, sin = self.rope_cos[pos], self.rope_sin[pos]
        for l in range(self.qkv.shape[0]):
            x = rms_norm(h, self.attn_ln[l], self.eps)
            qkv = F.linear(x, self.qkv[l])
            q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
            q = rope_interleaved(q.view(1, 1, Hq, D), cos, sin).to(h.dtype)
            k = rope_interleaved(k.view(1, 1, Hkv, D), cos, sin).to(h.dtype)
            self.k_cache[l, :, pos] = k[:, 0]
            self.v_cache[l, :, pos] = v.view(1, Hkv, D)
            kk = self.k_cache[l, :, : pos + 1].transpose(1, 2)  # [1, Hkv, T, D]
            vv = self.v_cache[l, :, : pos + 1].transpose(1, 2)
            attn = F.scaled_dot_product_attention(
                q.transpose(1, 2), kk, vv, is_causal=False, enable_gqa=True
            )
            attn = attn.transpose(1, 2).reshape(1, 1, Hq * D)
            h = h + F.linear(attn, self.o[l])
            x = rms_norm(h, self.mlp_ln[l], self.eps)
            prod = F.silu(F.linear(x, self.gate[l])) * F.linear(x, self.up[l])
            h = h + F.linear(prod, self.down[l])
        return h.reshape(-1)

    @torch.no_grad()
    def logits_from_hidden(self, hidden: Tensor) -> Tensor:
        x = rms_norm(hidden.reshape(1, 1, -1), self.final_norm, self.eps)
        return F.linear(x, self.head).reshape(-1)

    @torch.no_grad()
    def decode_token(self, token_id: int, pos: int) -> Tensor:
        """Embed ``token_id``, run one step at position ``pos``, return logits ``[V]``."""
        return self.logits_from_hidden(self.decode_hidden(self.embed[token_id], pos))


    @torch.no_grad()
    def decode_token_exact(self, token_id: int, pos: int) -> Tensor:
        """The same step in float32 throughout: bf16 weights and cache values, no intermediate
        rounding, nothing written back.  Not a reference path: it measures how far the bf16
        reference path itself sits from exact arithmetic at a given depth (its noise floor).
        Random-init networks amplify every rounding from layer to layer, so two faithful
        bf16 implementations drift apart with depth by about this much."""
        f32 = torch.float32
        h = self.embed[token_id].reshape(1, 1, -1).to(f32)
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        cos, sin = self.rope_cos[pos], self.rope_sin[pos]

        def norm(x, w):
            return w.to(f32) * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps))

        def lin(x, w):
            return F.linear(x, w.to(f32))

        for l in range(self.qkv.shape[0]):
            qkv = lin(norm(h, self.attn_ln[l]), self.qkv[l])
            q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
            q = rope_interleaved(q.view(1, 1, Hq, D), cos, sin)
            k = rope_interleaved(k.view(1, 1, Hkv, D), cos, sin)
            kk = torch.cat([self.k_cache[l, :, :pos].to(f32), k], dim=1).transpose(1, 2)
            vv = torch.cat([self.v_cache[l, :, :pos].to(f32), v.view(1, 1, Hkv, D)], dim=1).transpose(1, 2)
            attn = F.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, is_causal=False, enable_gqa=True)
            h = h + lin(attn.transpose(1, 2).reshape(1, 1, Hq * D), self.o[l])
            x = norm(h, self.mlp_ln[l])
            h = h + lin(F.silu(lin(x, self.gate[l])) * lin(x, self.up[l]), self.down[l])
        return lin(norm(h, self.final_norm), self.head).reshape(-1)


def parity_metrics(test: Tensor, ref: Tensor) -> dict:
    """The acceptance metrics for one step of logits.

    ``max_rel`` is ``max|test - ref| / max|ref|``; ``cosine`` is the cosine
    similarity; ``top2_margin`` is the gap between the reference's two largest
    logits, and ``argmax_equal`` whether both pick the same token.
    """
    a, b = test.float().flatten().cpu(), ref.float().flatten().cpu()
    top2 = torch.topk(b, 2).values
    top = float(top2[0].abs().clamp_min(1e-30))
    return {
        "max_rel": float((a - b).abs().max() / b.abs().max().clamp_min(1e-12)),
        "cosine": float(F.cosine_similarity(a, b, dim=0)),
        "top2_margin": float(top2[0] - top2[1]),
        # spacing of bf16 values (8 significant bits) at the largest logit
        "top_bf16_step": 2.0 ** (math.floor(math.log2(top)) - 7),
        "argmax_equal": bool(a.argmax() == b.argmax()),
    }


MAX_REL_TOL = 2e-2
COSINE_TOL = 0.999
MARGIN_TOL = 1e-2


def depth_aware_tolerance(oracle_logits: Tensor, exact_logits: Tensor) -> tuple[float, float, float]:
    """(max_rel, cosine, argmax margin) bounds for a step whose network is deep enough that the
    bf16 reference path itself misses the stated tolerance against exact arithmetic.

    ``exact_logits`` come from :meth:`TorchReferenceModel.decode_token_exact`.  The distance
    between two independent bf16 implementations is about sqrt(2) times the distance of one of
    them from exact arithmetic; the bound allows twice the oracle's own distance and never
    less than the stated tolerance (which therefore still applies wherever the reference
    path itself can meet it: shallow networks, all bisecting tests).  Likewise the argmax
    must agree wherever the oracle's top-2 margin exceeds twice the largest absolute error
    of the oracle's own logits (two candidates closer than that are ordered by rounding).
    """
    floor = parity_metrics(oracle_logits, exact_logits)
    abs_err = float((oracle_logits.float().flatten().cpu() - exact_logits.float().flatten().cpu()).abs().max())
    return (
        max(MAX_REL_TOL, 2.0 * floor["max_rel"]),
        min(COSINE_TOL, 1.0 - 4.0 * (1.0 - floor["cosine"])),
        max(MARGIN_TOL, 2.0 * abs_err),
    )


def assert_logits_parity(test: Tensor, ref: Tensor, what: str = "", exact: Tensor | None = None):
    """Stated tolerance; with ``exact`` (float32 restatement of the same step) the
    depth-aware bound of :func:`depth_aware_tolerance`."""
    m = parity_metrics(test, ref)
    max_rel_tol, cosine_tol, margin_tol = (
        (MAX_REL_TOL, COSINE_TOL, MARGIN_TOL) if exact is None else depth_aware_tolerance(ref, exact)
    )
    m["max_rel_tol"], m["cosine_tol"], m["margin_tol"] = max_rel_tol, cosine_tol, margin_tol
    assert m["max_rel"] <= max_rel_tol, f"{what}: max rel err {m['max_rel']:.4g} > {max_rel_tol:.4g}"
    assert m["cosine"] >= cosine_tol, f"{what}: cosine {m['cosine']:.6f} < {cosine_tol:.6f}"
    if m["top2_margin"] > margin_tol:
        assert m["argmax_equal"], f"{what}: argmax differs with margin {m['top2_margin']:.4g}"
    return m
