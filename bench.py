"""Decode benchmark of the resident decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config qwen3-8b|tiny]

Workload (N = 1): Qwen3-8B architecture, random-init BF16 weights ~N(0, 0.02) seed 0,
512-token seeded prompt, batch 1 greedy decode.  A "step" is one decoded token
(one replay of the resident step).  Prints ONE JSON line on rank 0.

  value     decode tok/s from CUDA events on the session stream around K graph replays,
            inputs (weights, KV, previous token) resident in HBM
  e2e       the same metric through the C ABI the way a streaming server calls it:
            one session_advance(steps=1) per token, host wall clock, device->host copy
            of the token slot and a stream synchronise inside every step
  roofline  the projection kernel (all five shapes): algorithmic weight+vector bytes
            per token / its summed device time per token, from an event-per-launch
            pass run after the timed region
  cpu_baseline / --impl reference: the CPU restatement of the reference decoder on
            the host cores (bounded sample)
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "Qwen3-8B-arch BF16 batch-1 decode tok/s"
# DRAM bytes (read + write) of the projection kernel's launches of one Qwen3-8B token, from the ncu
# capture summarised in profiles/projection_stream_kernel_qwen3_8b_shapes.md:
# 36 x (QKV 50.41 + O 33.63 + gate/up 205.18 + down 104.43 MB) + lm_head 1248.89 MB.
NCU_PROJECTION_TRAFFIC_PER_TOKEN = 36 * (50.41e6 + 33.63e6 + 205.18e6 + 104.43e6) + 1248.89e6
UNIT = "tok/s"


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
        return {"hbm_gbs": float(peaks["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.gpu_index = gpu_index
        self.lines: list[str] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def workload(name: str, layers: int = 0, prompt_tokens: int = 0):
    import dataclasses
    from nerva_b200 import synth
    cfg = synth.TINY_QWEN3 if name == "tiny" else synth.QWEN3_8B
    if layers > 0:       # profiler captures: same kernels and shapes, fewer layers resident
        cfg = dataclasses.replace(cfg, layers=layers, name=f"{cfg.name} cut to {layers} layers")
    if prompt_tokens > 0:
        cfg = dataclasses.replace(cfg, prompt_tokens=prompt_tokens)
    return cfg


def config_block(cfg, gpus: int, extra: dict | None = None) -> dict:
    block = {
        "workload": f"{cfg.name}: {cfg.layers} layers, hidden {cfg.hidden}, {cfg.heads}q/{cfg.kv_heads}kv heads, "
                    f"head_dim {cfg.head_dim}, intermediate {cfg.intermediate}, vocab {cfg.vocab}; batch 1, "
                    f"{cfg.prompt_tokens}-token seeded prompt, greedy decode",
        "weights": "random-init bf16 ~N(0,0.02) seed 0, unit norm weights, untied lm_head (synthetic)",
        "bytes_per_token": cfg.projection_bytes_per_token(),
        "l2": "each step streams the full weight set (far larger than the 126 MB L2); no flush needed",
        "parallelism": "single GPU" if gpus == 1 else
                       f"tp{gpus}: QKV, gate/up, lm_head split by rows, O and down by columns; partial sums "
                       f"exchanged inside the projection kernels over NVLink peer memory",
    }
    if extra:
        block.update(extra)
    return block


def cpu_decode_sample(ck, cfg, budget_s: float, max_tokens: int, prompt_len: int = 2):
    """Times the CPU restatement of the reference decoder (oracle, CPU contract) on a
    short prompt: returns (tok/s over the decode tokens, tokens timed, threads)."""
    from nerva_b200 import synth
    from oracle import oracle as O
    dec = O.Decoder(ck, prompt_len + max_tokens + 1, mode=O.MODE_CPU)
    prompt = synth.prompt_ids(cfg, count=prompt_len)
    for t in prompt[:-1]:
        dec.step(int(t), want_logits=False)
    token = int(prompt[-1])
    done, elapsed = 0, 0.0
    while done < max_tokens and (done == 0 or elapsed + elapsed / done < budget_s):
        t0 = time.perf_counter()
        logits = dec.step(token)
        token = O.argmax(logits, O.MODE_CPU)
        elapsed += time.perf_counter() - t0
        done += 1
    threads = O.lib().oracle_get_threads()
    dec.close()
    return done / elapsed, done, threads


def run_reference(args, cfg) -> dict:
    """The reference's own CPU implementation of the path (the C restatement of its
    Rust decoder; the Rust original cannot be compiled on this image), on all host
    threads.  Each step is one decoded token of the same model; steps stop early
    when the wall-clock budget is spent."""
    from nerva_b200 import ops, synth
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    budget = float(os.environ.get("NERVA_REFERENCE_BUDGET_S", "150"))
    warm_rate, _, threads = cpu_decode_sample(ck, cfg, budget_s=0.0, max_tokens=max(1, min(args.warmup, 1)))
    rate, done, threads = cpu_decode_sample(ck, cfg, budget_s=budget, max_tokens=args.steps)
    sample = (f"{done} of {args.steps} requested decode steps of the full model after a 2-token prompt "
              f"(stops at a {budget:.0f} s budget), {threads} threads")
    return {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus,
        "steps": done, "warmup": 1, "ms_per_step": 1000.0 / rate, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_block(cfg, 1),
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def run_ours(args, cfg, rank: int, world: int) -> dict:
    from nerva_b200 import build, ops, synth
    from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
    build.build()
    if args.timeline:
        os.environ["NERVA_B200_TIMELINE"] = "1"  # read when the session is created
    t0 = time.perf_counter()
    if world > 1:
        # tensor parallel: this rank generates and holds only its slices of the model
        ck = synth.dense_checkpoint_shard(cfg, rank, world, block_fill=ops.synth_normal_bf16_block,
                                          fill=ops.synth_normal_bf16)
    else:
        ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    gen_s = time.perf_counter() - t0
    prompt = synth.prompt_ids(cfg)
    profile_steps = 4
    timeline_steps = 10 if args.timeline else 0
    max_context = cfg.prompt_tokens + 1 + args.warmup + 2 * args.steps + profile_steps + timeline_steps + 8
    t0 = time.perf_counter()
    session = CudaHfDecodeSequenceSession(ck, max_context, engine=args.engine)
    if session.status != SmokeStatus.OK:
        raise RuntimeError(f"session create failed: {session.status} {session.error}")
    if world > 1:
        from nerva_b200 import tp
        tp.connect(session)
    create_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    start, loop = CudaHfDecodeSequenceLoop.start(session, prompt)
    if start.status != SmokeStatus.OK:
        raise RuntimeError(f"session start failed: {start.error}")
    prefill_s = time.perf_counter() - t0
    first = loop.advance(1)                      # the token the prefill produced (no replay)
    warm = loop.advance(max(args.warmup, 3))     # untimed warm-up replays
    if warm.status != SmokeStatus.OK:
        raise RuntimeError(f"warm-up failed: {warm.error}")

    sync = _barrier_fn(world)
    clocks = ClockSampler(int(os.environ.get("NERVA_GPU_INDEX", "0")))
    clocks.start()
    sync()
    timed = loop.advance(args.steps)             # K graph replays, timed by CUDA events on the session stream
    sync()
    if timed.status != SmokeStatus.OK or len(timed.tokens) != args.steps:
        raise RuntimeError(f"timed advance failed: {timed.error}")
    device_s = timed.device_elapsed_ns * 1e-9
    # end to end: one C-ABI call per token, host clock, D2H of the slot + synchronise each step
    t0 = time.perf_counter()
    e2e_tokens = 0
    for _ in range(args.steps):
        out = loop.advance(1)
        e2e_tokens += len(out.tokens)
    e2e_s = time.perf_counter() - t0
    clock_info = clocks.stop()
    timeline = None
    if args.timeline:
        # %globaltimer stamps written by the kernels themselves during ordinary graph replays
        acc = None
        for _ in range(timeline_steps):
            loop.advance(1)
            t = session.read_timeline().astype(np.int64)[:5 * cfg.layers].reshape(cfg.layers, 5, 8)
            rel = (t - t[:, 0, 0][:, None, None]).astype(np.float64)
            acc = rel if acc is None else acc + rel
            period = float((t[1:, 0, 0] - t[:-1, 0, 0]).mean()) / 1e3
        mean = (acc / timeline_steps)[1:-1].mean(axis=0) / 1e3 if cfg.layers > 2 else (acc / timeline_steps).mean(axis=0) / 1e3
        cols = ["entry", "after_wait", "after_prologue", "exit", "last_entry", "last_after_wait", "last_after_prologue",
                "last_exit"]
        timeline = {"layer_period_us": period, "columns": cols,
                    "us_since_qkv_entry": {name: [round(float(v), 2) for v in mean[i]]
                                           for i, name in enumerate(("qkv", "attention", "o", "gate_up", "down"))}}
    # per-kernel pass: events between launch groups, un-captured
    prof = session.profile_steps(profile_steps)
    session.destroy()

    device_s = _max_over_ranks(device_s, world)
    e2e_s = _max_over_ranks(e2e_s, world)
    proj_ns = sum(prof[k]["ns"] for k in ("qkv", "o", "gate_up", "down", "lm_head")) / profile_steps
    proj_launches = sum(prof[k]["launches_per_step"] for k in ("qkv", "o", "gate_up", "down", "lm_head"))
    # per GPU: this rank's weight slices + bf16 vectors
    bytes_per_token = ck.config.projection_bytes_per_token() + 2 * cfg.hidden * (3 * cfg.layers + 1)
    peaks = measured_peaks()
    achieved = bytes_per_token / (proj_ns * 1e-9) / 1e9
    kernel_name = "projection_stream_kernel (QKV, O, gate-up, down, lm_head)"
    kernel_us = proj_ns / 1e3
    if args.engine == 1:
        # one kernel per token: its launch duration is the event-timed step itself; its
        # algorithmic bytes add the KV rows read at the mean timed context and the KV row written
        mean_ctx = cfg.prompt_tokens + 1 + max(args.warmup, 3) + args.steps / 2
        kv_bytes = cfg.layers * 2 * cfg.kv_hidden * 2 * (mean_ctx + 1)
        bytes_per_token = bytes_per_token + int(kv_bytes)
        proj_launches = 1
        kernel_name = "decode_step_kernel (whole step: projections + attention + sampling)"
        kernel_us = 1e6 * device_s / args.steps
        achieved = bytes_per_token / (device_s / args.steps) / 1e9
    value = args.steps / device_s  # all ranks decode the same sequence together
    result = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": 1000.0 * device_s / args.steps, "higher_is_better": True,
        "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_block(cfg, world, {"timed_context": f"{cfg.prompt_tokens + 1 + max(args.warmup, 3)}.."
                                                              f"{cfg.prompt_tokens + 1 + max(args.warmup, 3) + args.steps}"}),
        "clocks": clock_info,
        "e2e": {"value": e2e_tokens / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 44,
                "note": "session_advance(steps=1) per token with host buffers; the ABI keeps the previous token on "
                        "the device, so a step has no host input; the prompt (4 B/token) is copied once in "
                        "session_start"},
        "gpu_launches": int(timed.kernel_launches),
        "roofline": {
            "bound": "hbm", "kernel": kernel_name,
            "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "peak_source": peaks["source"],
            "traffic": NCU_PROJECTION_TRAFFIC_PER_TOKEN if (world == 1 and cfg.name == "qwen3-8b") else None,
            "traffic_unit": "DRAM bytes per token over the same launches as bytes_per_token (ncu, see profiles/)",
            "launches_per_token": proj_launches, "bytes_per_token": bytes_per_token,
            "us_per_token": kernel_us, "engine": args.engine,
            "whole_step_frac": (bytes_per_token * args.steps / device_s / 1e9) / peaks["hbm_gbs"],
        },
        "profile_us_per_token": {k: v["ns"] / profile_steps / 1e3 for k, v in prof.items()},
        "setup_s": {"generate_weights": gen_s, "session_create": create_s, "prefill_by_decode": prefill_s},
        "graph_nodes": int(timed.graph_nodes),
        "token_hash": f"{timed.observed_token_hash:016x}",
    }
    if timeline is not None:
        result["timeline"] = timeline
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, done, threads = cpu_decode_sample(ck, cfg, budget_s=float(os.environ.get("NERVA_CPU_BUDGET_S", "20")),
                                                max_tokens=8)
        result["cpu_baseline"] = {
            "value": rate, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{done} decode steps of the full model after a 2-token prompt (CPU restatement of the "
                      f"reference decoder, row-parallel mat-vec)"}
    return result


def run_operator_workloads(kind: str) -> None:
    """Per-operator sweeps (isolated projection shapes, long-context attention) through the per-op C ABI (host buffers in,
    device time per launch out, L2 flushed between launches).  One JSON line per case."""
    from nerva_b200 import build, ops, synth
    build.build()
    peak = measured_peaks()
    if kind == "linear":
        shapes = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288),
                  ("lm_head", 151936, 4096)]
        for name, rows, cols in shapes:
            w = ops.synth_normal_bf16(0, 77, rows * cols, 0.02)
            for m in (1, 4, 16, 64):
                x = ops.synth_normal_bf16(0, synth.T_ACTIVATION, m * cols, 1.0)
                _, ns = ops.projection(w, x, rows, cols, tokens=m, warmup=3, iterations=10)
                nbytes = 2 * rows * cols + 2 * m * cols + 4 * m * rows
                gbs = nbytes / ns
                print(json.dumps({"workload": "decode-linear", "shape": name, "N": rows, "K": cols, "M": m,
                                  "us": ns / 1e3, "algorithmic_bytes": nbytes, "GB/s": gbs,
                                  "frac_of_measured_hbm": gbs / peak["hbm_gbs"],
                                  "note": "M > 1 re-streams the weights once per token (no skinny-GEMM kernel yet)"
                                  if m > 1 else "weight-streaming GEMV"}), flush=True)
        return
    heads, kv_heads, d = 32, 8, 128
    for batch in (1, 8):
        for context in (8192, 32768, 131072):
            pages = (context + 15) // 16
            n = batch * pages * 16 * kv_heads * d
            k = ops.synth_normal_bf16(0, synth.layer_tensor_id(0, synth.L_K), n, 1.0)
            v = ops.synth_normal_bf16(0, synth.layer_tensor_id(0, synth.L_V), n, 1.0)
            table = np.stack([synth.permutation(b, synth.T_PAGE_TABLE, pages) for b in range(batch)])
            q = synth.normal_f32(0, synth.layer_tensor_id(0, synth.L_Q), batch * heads * d, 1.0)
            _, ns = ops.gqa_decode_attention(q, k, v, table, batch, context, heads, kv_heads, d, warmup=3,
                                             iterations=10)
            nbytes = batch * (4096 * context + pages * 4 + heads * d * 4 * 2)
            gbs = nbytes / ns
            print(json.dumps({"workload": "long-context GQA decode attention", "batch": batch, "context": context,
                              "heads": heads, "kv_heads": kv_heads, "head_dim": d, "us": ns / 1e3,
                              "algorithmic_bytes": nbytes, "GB/s": gbs,
                              "frac_of_measured_hbm": gbs / peak["hbm_gbs"],
                              "pages": "16-token pages placed by a seeded Fisher-Yates permutation"}), flush=True)


def _barrier_fn(world: int):
    if world == 1:
        return lambda: None
    import torch.distributed as dist
    return dist.barrier


def _max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="qwen3-8b", choices=["qwen3-8b", "tiny"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--engine", type=int, default=0, choices=[0, 1],
                    help="0: one kernel per operator in a CUDA graph; 1: the whole-step kernel")
    ap.add_argument("--layers", type=int, default=0,
                    help="cut the model to this many layers (profiler captures only; not a bench line)")
    ap.add_argument("--prompt-tokens", type=int, default=0, help="override the prompt length")
    ap.add_argument("--workload", default="decode", choices=["decode", "linear", "attention"],
                    help="decode: the bench line; linear / attention: per-operator sweeps of the isolated "
                         "projection shapes and of long-context attention (one JSON line per case)")
    ap.add_argument("--timeline", action="store_true",
                    help="add the in-graph timeline (kernel-written %%globaltimer stamps, mean over layers)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload != "decode":
        if rank == 0:
            run_operator_workloads(args.workload)
        return
    cfg = workload(args.config, args.layers, args.prompt_tokens)
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args, cfg)), flush=True)
        return
    if world > 1:
        # one process per GPU; every GPU stays visible (the ranks map each other's exchange buffers)
        visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        os.environ["NERVA_GPU_INDEX"] = visible.split(",")[local] if visible else str(local)
        from nerva_b200 import tp
        tp.select_device(local)
        import torch.distributed as dist
        dist.init_process_group("gloo")
    result = run_ours(args, cfg, rank, world)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
