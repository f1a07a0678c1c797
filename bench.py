"""Benchmark of the decode hot path: batch-1 Llama decode through the megakernel.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one decoded token: embed the (teacher-forced, seeded) input token,
zero the barrier counters, launch the megakernel once, take the argmax.  At
N=1 the workload is the Llama-3.1-8B-architecture configuration (random-init
bf16 weights, KV cache prefilled to 1024 positions); at N>1 every rank runs an
independent replica of it (the 8B shape needs no sharding), so scaling is weak.

Rank 0 prints one JSON line.  ``value`` is tokens/s with all inputs resident in
HBM, timed with CUDA events around exactly K steps between barriers;
``e2e`` is the same metric with the token id coming from pinned host memory and
the produced token copied back to the host every step; ``roofline`` compares
the megakernel's average launch time against the measured HBM copy bandwidth;
``cpu_baseline`` times the CPU oracle on a bounded sample of the same workload.
``--impl reference`` times only that CPU path (the reference's algorithm on the
host cores) and prints the same kind of line.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "batch1_decode_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used when MEASURED_PEAKS.json is absent

# DRAM traffic of one megakernel launch relative to its algorithmic bytes, from the ncu capture
# summarised in profiles/megakernel_llama8b_4layers_ncu_full.md: (2.855 GB read + 0.034 GB written)
# against 2.796 GB algorithmic on the 4-layer case; traffic grows in proportion to the layers
# streamed, so the full launch is scaled by the same ratio.
NCU_TRAFFIC_RATIO = (2.8553e9 + 0.0336e9) / 2.7955e9

WORKLOADS = {
    # tp=False: every rank runs an independent replica; tp=True: the ranks shard one model
    "llama-3.1-8b": dict(preset="llama_3_1_8b", prefill=1024, tp=False),
    "llama-3.2-1b": dict(preset="llama_3_2_1b", prefill=32, tp=False),
    "llama-3.1-70b": dict(preset="llama_3_1_70b", prefill=2048, tp=True),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama-3.1-8b", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=0, help="override depth (profiling small cases)")
    ap.add_argument("--prefill", type=int, default=0)
    ap.add_argument("--sched", default="rr")
    ap.add_argument("--attn-partitions", type=int, default=0, help="0 = pick from the length")
    ap.add_argument("--no-coalesce-o-proj", action="store_true")
    ap.add_argument("--balance", action="store_true",
                    help="timeline-model builder with pinned SMs instead of the even split + --sched")
    ap.add_argument("--barrier-fill", type=int, default=0,
                    help="experiment: preset all barrier counters (waits pass at once; results are garbage)")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="replay one captured decode step per token instead of launching eagerly")
    ap.add_argument("--tp-exchange", default="peer", choices=["peer", "nccl"],
                    help="tensor-parallel workloads: all-reduce inside the kernel over peer memory "
                         "(one launch per token) or NCCL between 2L+1 launches")
    ap.add_argument("--tp-chunks", type=int, default=0, help="chunks per in-kernel all-reduce (0 = H / 1024)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def model_config(args):
    from megakernels_b200.llama import LlamaConfig

    w = WORKLOADS[args.workload]
    overrides = {"num_hidden_layers": args.layers} if args.layers else {}
    cfg = getattr(LlamaConfig, w["preset"])(**overrides)
    prefill = args.prefill or w["prefill"]
    return cfg, prefill


def algorithmic_bytes_per_token(cfg, seq_len: int, tp: int = 1) -> dict:
    """Bytes one GPU must move per decoded token: every bf16 matrix of its shard once
    (layers split over ``tp`` ranks, LM head replicated), norms, KV read + append."""
    H, I, L, D = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers, cfg.head_dim
    Hq, Hkv, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.vocab_size
    per_layer = ((Hq + 2 * Hkv) * D * H + H * Hq * D + 3 * I * H) * 2 // tp
    weights = L * per_layer + V * H * 2
    norms = (2 * L + 1) * H * 2
    kv_row = 2 * Hkv * D * 2 * L // tp
    return dict(weights=weights, norms=norms, kv=kv_row * seq_len + kv_row)


def hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = (
        "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index: int):
        self.index = index
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = self.rows
        mhz = sorted(float(r[0]) for r in rows if r[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {
            "sm_mhz": mhz[len(mhz) // 2] if mhz else None,
            "sm_max_mhz": float(rows[0][1]) if rows and rows[0][1].replace(".", "").isdigit() else None,
            "reasons": reasons,
            "samples": len(rows),
        }


# --------------------------------------------------------------------------- #
# CPU path (oracle port of the reference's torch decode step)
# --------------------------------------------------------------------------- #
def time_cpu_path(cfg, prefill: int, tokens: int, sample_layers: int, budget_s: float = 25.0):
    """Time the CPU oracle on ``sample_layers`` layers + the LM head; scale to full depth."""
    import dataclasses

    from megakernels_b200.llama import LlamaForCausalLM
    from megakernels_b200.model_types import ExtraModelConfig
    from oracle.llama_ref import TorchReferenceModel

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    small = dataclasses.replace(cfg, num_hidden_layers=sample_layers)
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=prefill + tokens + 1)
    model = LlamaForCausalLM.from_random(small, extra, device="cpu", seed=0)
    gen = torch.Generator().manual_seed(2)
    for c in model.stacked_kv_cache:
        c[:, :, :prefill] = torch.randn(c[:, :, :prefill].shape, generator=gen).to(c.dtype)
    ref = TorchReferenceModel(model)
    ref.load_kv(*model.stacked_kv_cache)
    ids = torch.randint(0, cfg.vocab_size, (tokens + 1,), generator=torch.Generator().manual_seed(3))
    per_token = []
    t_begin = time.perf_counter()
    for i in range(tokens + 1):
        t0 = time.perf_counter()
        h = ref.decode_hidden(ref.embed[int(ids[i])], prefill + i)
        t1 = time.perf_counter()
        ref.logits_from_hidden(h)
        t2 = time.perf_counter()
        if i > 0:  # first token warms the thread pool
            per_token.append((t1 - t0) * (cfg.num_hidden_layers / sample_layers) + (t2 - t1))
        if time.perf_counter() - t_begin > budget_s and len(per_token) >= 2:
            break
    sec = sum(per_token) / len(per_token)
    return dict(
        value=1.0 / sec,
        unit=UNIT,
        cores=cores,
        kind="port",
        sample=(
            f"oracle/llama_ref.py torch decode step on {sample_layers} of {cfg.num_hidden_layers} layers "
            f"+ LM head, {len(per_token)} tokens at KV length {prefill}; layer time scaled by "
            f"{cfg.num_hidden_layers / sample_layers:g}"
        ),
    ), sec


def run_reference_arm(args):
    cfg, prefill = model_config(args)
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_layers = min(2, cfg.num_hidden_layers)
    # every step is one decoded token of the sample; K + W tokens in total
    tokens = max(2, min(args.steps + args.warmup, 64))
    base, sec = time_cpu_path(cfg, prefill, tokens, sample_layers, budget_s=120.0)
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": base["value"],
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": sec * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"{args.workload} batch-1 decode, KV prefill {prefill}", "inputs": "larger than L2"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def build_engine(args, device, tp_size=1, tp_rank=0, group=None):
    from megakernels_b200.demos.latency.scheduler import (
        LatencyScheduleOptions,
        pick_num_attention_partitions,
    )
    from megakernels_b200.dispatch import make_mk_interpreter, make_schedule_builder
    from megakernels_b200.generators import MK_Generator, TP_MK_Generator, TP_Peer_MK_Generator
    from megakernels_b200.llama import LlamaForCausalLM
    from megakernels_b200.model_types import ExtraModelConfig
    from megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    cfg, prefill = model_config(args)
    total = prefill + args.steps + args.warmup + 8
    extra = ExtraModelConfig(
        interleave_rope=True, max_len_override=total, tp_size=tp_size, tp_rank=tp_rank, tp_group=group
    )
    model = LlamaForCausalLM.from_random(cfg, extra, device=device, seed=0, draw_on="device")
    gen = torch.Generator(device=device).manual_seed(2 + tp_rank)
    for c in model.stacked_kv_cache:
        c[:, :, :prefill] = torch.randn(c[:, :, :prefill].shape, generator=gen, device=device).to(c.dtype)
    n_part = args.attn_partitions or pick_num_attention_partitions(
        prefill, args.steps + args.warmup, device, model.num_kv_heads(), min_chunk_size=128
    )
    balance = args.balance
    peer = tp_size > 1 and args.tp_exchange == "peer"
    options = LatencyScheduleOptions(
        num_attention_partitions=n_part, coalesce_o_proj=not args.no_coalesce_o_proj, balance=balance,
        # chunks of 1024 elements: one pair per consumer thread, a multiple of the TP degree
        tp_all_reduce_chunks=(args.tp_chunks or max(tp_size, cfg.hidden_size // 1024)) if peer else 0,
    )
    if balance:
        args.sched = "hint"
    schedule = make_schedule_builder("latency", options).build(model)
    schedule.globs.pos_id = prefill
    interp = make_mk_interpreter("latency")
    if peer:
        tensorize_instructions(schedule.globs, assign_to_sms(args.sched, schedule=schedule))
        generator = TP_Peer_MK_Generator(model, interp, schedule, group=group)
        launches_per_step = 1
    elif tp_size > 1:
        generator = TP_MK_Generator(model, interp, schedule, group=group, sched=args.sched)
        launches_per_step = len(generator.segments)
    else:
        tensorize_instructions(schedule.globs, assign_to_sms(args.sched, schedule=schedule))
        generator = MK_Generator(model, interp, schedule, barrier_fill_val=args.barrier_fill)
        launches_per_step = 1
    info = dict(attn_partitions=n_part, instructions=len(schedule.get_linear_instructions()),
                launches_per_step=launches_per_step)
    return cfg, prefill, model, schedule, generator, info


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    distributed = world > 1
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    tp = WORKLOADS[args.workload]["tp"] and world > 1
    if WORKLOADS[args.workload]["tp"] and world == 1:
        raise SystemExit(f"{args.workload} is the tensor-parallel workload: launch it on 2, 4 or 8 GPUs")
    log("building model and schedule")
    cfg, prefill, model, schedule, gen, info = build_engine(
        args, device, tp_size=world if tp else 1, tp_rank=rank if tp else 0
    )
    gen_holder = [gen]
    log(f"engine ready: {info}")
    K, W = args.steps, args.warmup
    ids = torch.randint(0, cfg.vocab_size, (W + K,), generator=torch.Generator().manual_seed(3))
    ids_dev = ids.to(device).view(-1, 1, 1)
    # 2L+1 launches per token (NCCL exchange) are launch-bound without a graph
    use_graph = args.cuda_graph or (tp and args.tp_exchange == "nccl")

    # ---- warm-up ----------------------------------------------------------- #
    for i in range(min(W, 3)):
        gen.run(ids_dev[i], pos_id=prefill + i)
    gen.check()
    log("eager warm-up done")
    if use_graph:
        gen.enable_cuda_graph(warmup_pos=prefill)
        log("graph captured")
    for i in range(W):
        gen.run(ids_dev[i], pos_id=prefill + i)
    gen.check()

    # ---- device-resident timing: exactly K steps between barriers -------- #
    log("warm-up done, timing")
    sampler = ClockSampler(local_rank)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launch_events = []
    interp = gen.interpreter
    globs = schedule.globs
    embed = model.model.embed_tokens.embed_tokens.weight
    barrier()
    log("barrier passed")
    sampler.start()
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` see only the timed region
    start.record()
    if use_graph:
        for i in range(K):
            gen.run(ids_dev[W + i], pos_id=prefill + W + i)
    else:
        for i in range(K):
            # the body of MK_Generator.run, with events around the kernel launch
            globs.hidden_states[:] = embed[ids_dev[W + i]].reshape(-1)
            gen.fill()
            globs.pos_id = prefill + W + i
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gen.last_call = interp.interpret(globs)
            e1.record()
            launch_events.append((e0, e1))
            if globs.tp is not None:
                globs.tp.epoch_device.add_(1)  # as TP_Peer_MK_Generator._step does
            gen._next_token()  # the kernel's own argmax word (torch.argmax if that is switched off)
    end.record()
    torch.cuda.profiler.stop()
    log("timed steps enqueued")
    barrier()
    log("timed steps finished")
    clocks = sampler.stop()
    gen.check()
    elapsed_ms = start.elapsed_time(end)
    if launch_events:
        kernel_ms = sum(a.elapsed_time(b) for a, b in launch_events) / K
        kernel_scope = "megakernel launch"
    else:
        # inside a graph the launches cannot be bracketed: the roofline covers the whole step
        kernel_ms = elapsed_ms / K
        kernel_scope = "whole decode step (graph replay" + (", incl. all-reduces)" if tp else ")")

    # ---- end to end: token id from pinned host memory, produced token back to host ---- #
    e2e = None
    if not args.no_e2e:
        host_in = torch.empty(1, dtype=torch.long).pin_memory()
        host_out = torch.empty(1, dtype=torch.long).pin_memory()
        dev_in = torch.empty(1, 1, dtype=torch.long, device=device)
        pos0 = prefill + W  # re-decode the same positions: same work per step
        if not use_graph:
            # the public generator replays the whole step (embedding row, counter reset, megakernel,
            # argmax) as one CUDA graph; the device-timed loop above stays eager so that each
            # megakernel launch can be bracketed by events
            gen.enable_cuda_graph(warmup_pos=prefill)
        for i in range(3):
            host_in[0] = ids[W + i]
            dev_in.copy_(host_in.view(1, 1), non_blocking=True)
            host_out.copy_(gen.run(dev_in, pos_id=pos0 + i).view(-1), non_blocking=True)
            torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        for i in range(K):
            host_in[0] = ids[W + i]
            dev_in.copy_(host_in.view(1, 1), non_blocking=True)
            out = gen.run(dev_in, pos_id=pos0 + i)
            host_out.copy_(out.view(-1), non_blocking=True)
            torch.cuda.current_stream().synchronize()
            _ = int(host_out[0])
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        gen.check()
        e2e = e2e_s

    # ---- reduce over ranks ------------------------------------------------ #
    if distributed:
        t = torch.tensor([elapsed_ms, kernel_ms, e2e or 0.0], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, kernel_ms, e2e_max = t.tolist()
        e2e = e2e_max if e2e is not None else None

    if rank == 0:
        peak, peak_kind = hbm_peak()
        mid_len = prefill + W + K // 2
        nbytes = algorithmic_bytes_per_token(cfg, mid_len, tp=world if tp else 1)
        algo = sum(nbytes.values())
        achieved = algo / (kernel_ms * 1e-3) / 1e9
        replicas = 1 if tp else world  # a tensor-parallel job decodes one sequence
        line = {
            "metric": METRIC,
            "value": replicas * K / (elapsed_ms * 1e-3),
            "unit": UNIT,
            "n_gpus": world,
            "steps": K,
            "warmup": W,
            "ms_per_step": elapsed_ms / K,
            "higher_is_better": True,
            "scaling": "strong" if tp else "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": f"{args.workload} batch-1 decode, {cfg.num_hidden_layers} layers, KV prefill {prefill}, "
                            f"{K} teacher-forced steps"
                            + (f", tensor parallel over {world} GPUs ("
                               + ("in-kernel all-reduce over peer memory" if args.tp_exchange == "peer" else "NCCL all-reduce")
                               + " after o-proj and down-proj)" if tp
                               else (f", {world} independent replicas" if world > 1 else "")),
                "launch": "cuda graph replay" if use_graph else "eager",
                "e2e_launch": "cuda graph replay of the whole step",
                "inputs": "larger than L2 (weights re-streamed from HBM every step)",
                "sched": args.sched,
                **info,
            },
            "kernel_ms_per_launch": kernel_ms,
            "roofline_scope": kernel_scope,
            "roofline": {
                "bound": "hbm",
                "achieved": achieved,
                "peak": peak,
                "unit": "GB/s",
                "frac": achieved / peak,
                "peak_source": f"{peak_kind} copy bandwidth",
                "frac_of_nominal_8TBs": achieved / 8000.0,
                "weight_only_frac": (nbytes["weights"] / (kernel_ms * 1e-3) / 1e9) / peak,
                "algorithmic_bytes_per_launch": algo,  # per GPU and decoded token
                "traffic": algo * NCU_TRAFFIC_RATIO,
                "traffic_source": "ncu dram bytes of a 4-layer capture scaled to this launch",
            },
            "clocks": clocks,
            "gpu_launches": world * K * info["launches_per_step"],
        }
        if e2e is not None:
            line["e2e"] = {
                "value": replicas * K / e2e,
                "unit": UNIT,
                "h2d_bytes_per_step": 8,
                "d2h_bytes_per_step": 8,
                "ms_per_step": e2e / K * 1e3,
            }
        if world == 1 and not args.no_cpu_baseline:
            del model, schedule, gen
            torch.cuda.empty_cache()
            base, _ = time_cpu_path(cfg, prefill, tokens=6, sample_layers=min(2, cfg.num_hidden_layers))
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if distributed:
        # Tear down in a fixed order: captured graphs hold NCCL kernels, and destroying the
        # communicator underneath them was seen to block at interpreter exit.
        dist.barrier()
        torch.cuda.synchronize()
        if getattr(gen_holder[0], "_graph", None) is not None:
            gen_holder[0]._graph = None
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def log(msg: str):
    """Progress lines on stderr when MKB_BENCH_VERBOSE is set (stdout carries only the JSON line)."""
    if os.environ.get("MKB_BENCH_VERBOSE"):
        print(f"[bench {time.strftime('%H:%M:%S')} rank {os.environ.get('RANK', '0')}] {msg}",
              file=sys.stderr, flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
