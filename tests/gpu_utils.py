"""Helpers of the GPU parity tests: run the same instruction stream on the CPU
oracle and through the C-ABI CUDA library, on identical seeded inputs."""

from __future__ import annotations

import sys

import torch

from megakernels_b200.dispatch import make_mk_interpreter
from megakernels_b200.scheduler import assign_to_sms, tensorize_instructions
from oracle.python_vm import PyVM_Interpreter
from tests.oracle_utils import build_model, build_schedule, fill_kv

ACTIVATIONS = ("hidden_states", "post_ln_rope_q", "attn_out", "silu_out", "logits")


def make_pair(cfg, max_len, prefill, options=None, sched="rr", poison=True, **build_kw):
    """(cpu_model, cpu_schedule, gpu_model, gpu_schedule) on identical weights and KV."""
    cpu_model = build_model(cfg, max_len, device="cpu")
    fill_kv(cpu_model, prefill, poison=poison)
    gpu_model = build_model(cfg, max_len, device="cuda:0")
    for a, b in zip(gpu_model.stacked_kv_cache, cpu_model.stacked_kv_cache):
        a.copy_(b)
    cpu_sched = build_schedule(cpu_model, options, **build_kw)
    gpu_sched = build_schedule(gpu_model, options, **build_kw)
    tensorize_instructions(cpu_sched.globs, assign_to_sms(sched, schedule=cpu_sched))
    tensorize_instructions(gpu_sched.globs, assign_to_sms(sched, schedule=gpu_sched))
    return cpu_model, cpu_sched, gpu_model, gpu_sched


def run_cpu_step(cpu_model, cpu_sched, hidden, pos):
    g = cpu_sched.globs
    g.hidden_states[:] = hidden
    g.barriers.zero_()
    g.pos_id = pos
    PyVM_Interpreter().interpret(g, cpu_sched.get_linear_instructions())


_interp = None


def interpreter():
    global _interp
    if _interp is None:
        _interp = make_mk_interpreter("latency")
    return _interp


def run_gpu_step(gpu_sched, hidden, pos, **kw):
    g = gpu_sched.globs
    g.hidden_states[:] = hidden.to(g.hidden_states.device)
    g.vm_state.zero_()  # barrier counters and residual accumulators
    g.pos_id = pos
    call = interpreter().interpret(g, **kw)
    mk = sys.modules["mk_llama"]
    return mk.sync_status(call)


def rel_err(test: torch.Tensor, ref: torch.Tensor) -> float:
    a, b = test.float().cpu().flatten(), ref.float().cpu().flatten()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-12))


def tensor_of(g, name):
    """Activation tensor by name; the residual stream is the embedding plus the accumulators."""
    return g.residual_stream() if name == "hidden_states" else getattr(g, name)


def compare_globals(gpu_g, cpu_g, pos, names=ACTIVATIONS, tol=2e-2):
    """max|gpu - cpu| / max|cpu| per tensor; returns the dict, asserts the tolerance."""
    out = {}
    for name in names:
        out[name] = rel_err(tensor_of(gpu_g, name), tensor_of(cpu_g, name))
    out["k_new"] = rel_err(gpu_g.k_cache[:, 0, pos], cpu_g.k_cache[:, 0, pos])
    out["v_new"] = rel_err(gpu_g.v_cache[:, 0, pos], cpu_g.v_cache[:, 0, pos])
    bad = {k: v for k, v in out.items() if not v <= tol}
    assert not bad, f"tensors out of tolerance {tol}: {bad} (all: {out})"
    return out
