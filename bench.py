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
  roofline  the projection kernel (all five shapes): algorithmic weight+vector bytes per
            token / the time its launches are busy inside ordinary graph replays, net of
            overlap with their neighbours (kernel-written %globaltimer stamps of a fork of
            the session that shares the weights); `isolated_frac` is the same bytes over an
            event-per-launch pass outside the graph
  parity    the decoded tokens against the committed oracle stream of the same prompt
            (tests/golden/qwen3_8b.json): first diverging step and the oracle's margin there
  cpu_baseline / --impl reference: the CPU restatement of the reference decoder on
            the host cores (bounded sample at the same context)
  gpu_baseline (N = 1): the reference's own CUDA library (cuBLASLt projections), built from
            the reference checkout into oracle/_ref, decoding the same workload in a child
            process after everything else has been measured
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
# DRAM bytes (read + write) of the projection kernel's launches of one Qwen3-8B token.  NOT measured
# by a bench run (a profiler cannot sit inside the timed region): taken from the ncu capture
# summarised in profiles/projection_stream_kernel_qwen3_8b_shapes.md, per launch
# QKV 50.41 + O 33.63 + gate/up 205.18 + down 104.43 MB, lm_head 1248.89 MB.
NCU_PROJECTION_TRAFFIC_PER_TOKEN = 36 * (50.41e6 + 33.63e6 + 205.18e6 + 104.43e6) + 1248.89e6
NCU_TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, capture summarised in "
                      "profiles/projection_stream_kernel_qwen3_8b_shapes.md (not re-measured by this run)")
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
        self.lines: list[tuple[float, str]] = []
        self.proc = None
        self.thread = None
        self.begin = None

    def start(self, wait_s: float = 8.0):
        """Starts the sampling process and waits until its first sample has arrived (nvidia-smi takes a
        while to come up on a machine with many GPUs), so that a short timed region is not over before
        the first sample; the region itself begins at mark()."""
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()
        deadline = time.perf_counter() + wait_s
        while not self.lines and time.perf_counter() < deadline and self.proc.poll() is None:
            time.sleep(0.01)
        self.mark()

    def mark(self):
        """The load to be sampled starts now: earlier samples are dropped from the report."""
        self.begin = time.perf_counter()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def samples_since_mark(self) -> int:
        return sum(1 for t, _ in self.lines if self.begin is None or t >= self.begin)

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
        for stamp, line in self.lines:
            if self.begin is not None and stamp < self.begin:
                continue
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


MAX_EXTRA_CLOCK_STEPS = 512


def extra_clock_steps(timed_s: float, steps: int) -> int:
    """Untimed steps to run behind the timed and the end-to-end region (each `steps` long, about
    timed_s) so that the clock sampler, which reports every 50 ms, sees this load for about 0.35 s."""
    if timed_s <= 0 or steps <= 0:
        return 0
    missing = 0.35 - 2.0 * timed_s
    if missing <= 0:
        return 0
    return min(MAX_EXTRA_CLOCK_STEPS, int(missing / (timed_s / steps)) + 1)


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


def host_threads() -> int:
    """All host cores, whatever OMP_NUM_THREADS says (torch.distributed.run exports 1)."""
    return max(1, len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))


def cpu_decode_sample(ck, cfg, budget_s: float, max_tokens: int, warmup_tokens: int = 1):
    """Times the CPU restatement of the reference decoder (oracle, CPU contract) at the workload's
    context: the cache is positioned at the prompt length (patterned rows instead of a CPU prefill,
    which alone would take minutes; a decode step costs the same whatever the cached values are),
    then `warmup_tokens` untimed and up to `max_tokens` timed decode steps within `budget_s`.
    Returns (tok/s, tokens timed, threads)."""
    from nerva_b200 import synth
    from oracle import oracle as O
    threads = host_threads()
    O.lib().oracle_set_threads(threads)
    dec = O.Decoder(ck, cfg.prompt_tokens + warmup_tokens + max_tokens + 1, mode=O.MODE_CPU)
    dec.seek_for_timing(cfg.prompt_tokens)
    token = int(synth.prompt_ids(cfg, count=1)[0])
    for _ in range(warmup_tokens):
        token = O.argmax(dec.step(token), O.MODE_CUDA)
    done, elapsed = 0, 0.0
    while done < max_tokens and (done == 0 or elapsed + elapsed / done < budget_s):
        t0 = time.perf_counter()
        logits = dec.step(token)
        token = O.argmax(logits, O.MODE_CUDA)
        elapsed += time.perf_counter() - t0
        done += 1
    dec.close()
    return done / elapsed, done, threads


def cpu_sample_text(cfg, done: int, requested: int, threads: int) -> str:
    return (f"{done} of {requested} decode steps of the full {cfg.layers}-layer model at context "
            f"{cfg.prompt_tokens} (cache positioned there with patterned rows instead of a CPU prefill), "
            f"{threads} host threads, row-parallel mat-vec")


def run_reference(args, cfg) -> dict:
    """The reference's own CPU implementation of the path (the C restatement of its
    Rust decoder; the Rust original cannot be compiled on this image), on all host
    threads.  Each step is one decoded token of the same model at the same context; steps
    stop early when the wall-clock budget is spent.  Weights come from the oracle's own
    generator: this arm does not load the CUDA library."""
    from nerva_b200 import synth
    from oracle import oracle as O
    O.lib().oracle_set_threads(host_threads())
    ck = synth.dense_checkpoint(cfg, fill=O.synth_normal_bf16)
    budget = float(os.environ.get("NERVA_REFERENCE_BUDGET_S", "150"))
    rate, done, threads = cpu_decode_sample(ck, cfg, budget_s=budget, max_tokens=args.steps,
                                            warmup_tokens=max(1, min(args.warmup, 2)))
    sample = cpu_sample_text(cfg, done, args.steps, threads) + f"; stops at a {budget:.0f} s budget"
    return {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus,
        "steps": done, "warmup": max(1, min(args.warmup, 2)), "ms_per_step": 1000.0 / rate, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_block(cfg, args.gpus),
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def golden_stream(cfg):
    """The committed oracle stream of the headline workload, or None for other workloads."""
    path = os.path.join(ROOT, "tests", "golden", "qwen3_8b.json")
    if cfg.name != "qwen3-8b" or cfg.prompt_tokens != 512 or not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f)["cuda"]


def parity_block(cfg, tokens) -> dict:
    """Compares the decoded tokens (from the first generated one) with the oracle's stream."""
    golden = golden_stream(cfg)
    if golden is None:
        return {"reference": None, "note": "no committed oracle stream for this workload"}
    want = golden["tokens"]
    n = min(len(tokens), len(want))
    at = next((i for i in range(n) if int(tokens[i]) != int(want[i])), None)
    return {
        "reference": "tests/golden/qwen3_8b.json: CPU oracle, CUDA numeric contract, serial fp32 sums",
        "tokens_compared": n, "tokens_identical": n if at is None else at,
        "first_divergence_step": at,
        "margin_at_divergence": None if at is None else golden["top1_minus_top2"][at],
        "note": "after a divergence the two streams decode different sequences; a divergence is a tie when the "
                "oracle's top-1 minus top-2 margin there is below twice its own distance to itself under another "
                "fp32 summation order (0.185 at 36 layers)",
    }


def teacher_forced_parity(session, cfg, positions: int = 64) -> dict | None:
    """The session against the committed oracle stream position by position: it decodes freely until
    its token differs from the oracle's, then the request is restarted on the prompt plus the oracle's
    own tokens, so that every position is compared on the oracle's history.  A differing token is a
    near tie when the oracle's top-1 minus top-2 margin there is below the bound (twice the oracle's
    own distance to itself under another fp32 summation order, twice over) and the token is among the
    oracle's eight best."""
    from nerva_b200 import synth
    from nerva_b200.session import CudaHfDecodeSequenceLoop, SmokeStatus
    path = os.path.join(ROOT, "tests", "golden", "qwen3_8b.json")
    if cfg.name != "qwen3-8b" or cfg.prompt_tokens != 512 or not os.path.exists(path):
        return None
    with open(path) as f:
        golden = json.load(f)
    g = golden["cuda"]
    sweep = golden["depth_sweep"]
    self_distance = sweep["self_distance"][sweep["depths"].index(cfg.layers)] if cfg.layers in sweep["depths"] else None
    if self_distance is None:
        return None
    bound = max(2e-2, 2.0 * self_distance)
    idx = golden["sample_indices"]
    prompt = synth.prompt_ids(cfg)
    positions = min(positions, len(g["tokens"]))
    start, loop = CudaHfDecodeSequenceLoop.start(session, prompt)
    if start.status != SmokeStatus.OK:
        return {"error": start.error}
    equal, ties, outside, worst = 0, [], [], 0.0
    for i in range(positions):
        out = loop.advance(1)
        if out.status != SmokeStatus.OK or not out.tokens:
            return {"error": out.error}
        logits = session.read_logits()
        want = np.array(g["logit_samples"][i] + g["top8_value"][i], dtype=np.float32)
        got = np.concatenate([logits[idx], logits[g["top8_index"][i]]])
        worst = max(worst, float(np.abs(got - want).max()))
        if out.tokens[0] == g["tokens"][i]:
            equal += 1
            continue
        entry = {"position": i, "oracle_margin": g["top1_minus_top2"][i]}
        (ties if g["top1_minus_top2"][i] <= 2.0 * bound and out.tokens[0] in g["top8_index"][i] else outside).append(entry)
        if i + 1 < positions:
            restarted = np.concatenate([prompt, np.array(g["tokens"][:i + 1], dtype=np.uint32)])
            start, loop = CudaHfDecodeSequenceLoop.start(session, restarted)
            if start.status != SmokeStatus.OK:
                return {"error": start.error}
    return {"positions": positions, "tokens_equal": equal, "near_ties": ties, "outside_the_tie_rule": outside,
            "max_abs_logit_error_on_samples": worst, "logit_bound": bound, "oracle_self_distance": self_distance}


def timeline_busy_us(session, loop, cfg, steps: int) -> dict:
    """Per operator kind, the time its launches are busy inside ordinary graph replays, net of
    overlap: launches are walked in launch order and each is charged from max(its first stamp, the
    end of everything before it) to its last stamp.  Mean over `steps` replays, microseconds."""
    kinds = ("qkv", "attention", "o", "gate_up", "down")
    total = {k: 0.0 for k in kinds + ("lm_head",)}
    span = 0.0
    for _ in range(steps):
        out = loop.advance(1)
        if not out.tokens:
            raise RuntimeError("timeline step failed: " + out.error)
        t = session.read_timeline().astype(np.int64)
        covered = None
        first = None
        for node in range(5 * cfg.layers + 1):
            row = t[node]
            begin, end = int(min(row[0], row[4])), int(max(row[3], row[7]))
            if first is None:
                first = begin
            kind = "lm_head" if node == 5 * cfg.layers else kinds[node % 5]
            lo = begin if covered is None else max(begin, covered)
            if end > lo:
                total[kind] += (end - lo) / 1e3
            covered = end if covered is None else max(covered, end)
        span += (covered - first) / 1e3
    out = {k: v / steps for k, v in total.items()}
    out["step_span"] = span / steps
    return out


def gpu_baseline_child(args, cfg) -> dict:
    """Runs the reference's CUDA library on the same workload in a child process (its own CUDA
    context, nothing of this library on its path) and returns its JSON line."""
    lib_path = os.path.join(ROOT, "oracle", "_ref", "libnerva_ref_decode.so")
    if not os.path.exists(lib_path):
        return {"unavailable": "oracle/_ref/libnerva_ref_decode.so has not been built (needs the reference checkout)"}
    cmd = [sys.executable, os.path.abspath(__file__), "--workload", "reference-gpu", "--steps", str(min(args.steps, 64)),
           "--warmup", str(max(args.warmup, 3)), "--config", args.config]
    if args.layers:
        cmd += ["--layers", str(args.layers)]
    if args.prompt_tokens:
        cmd += ["--prompt-tokens", str(args.prompt_tokens)]
    try:
        done = subprocess.run(cmd, capture_output=True, text=True, timeout=float(os.environ.get("NERVA_GPU_BASELINE_S", "420")))
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference CUDA library did not finish within its time limit"}
    for line in reversed(done.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    return {"unavailable": f"no result line (rc {done.returncode}): {done.stderr.strip()[-300:]}"}


def run_reference_gpu(args, cfg) -> None:
    """The reference's CUDA decode library (cuBLASLt projections, its own kernels around them) on
    this workload: session_create with planned descriptors, session_start (its chunked cuBLAS
    prefill), warm-up, then `steps` graph replays timed by its own start/stop events."""
    from nerva_b200 import ffi, synth
    from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
    from oracle import oracle as O
    O.lib().oracle_set_threads(host_threads())
    library = ffi.load_abi_library(os.path.join(ROOT, "oracle", "_ref", "libnerva_ref_decode.so"))
    ck = synth.dense_checkpoint(cfg, fill=O.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    warm = max(args.warmup, 3)
    t0 = time.perf_counter()
    session = CudaHfDecodeSequenceSession(ck, cfg.prompt_tokens + 1 + warm + args.steps + 4, use_descriptors=True,
                                          library=library)
    if session.status != SmokeStatus.OK:
        print(json.dumps({"unavailable": f"reference session_create failed: cuda_error "
                                         f"{session.create_result.cuda_error}, stage {session.create_result.failure_stage}"}))
        return
    create_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    start, loop = CudaHfDecodeSequenceLoop.start(session, prompt)
    if start.status != SmokeStatus.OK:
        print(json.dumps({"unavailable": f"reference session_start failed: cuda_error {start.cuda_error}"}))
        return
    prefill_s = time.perf_counter() - t0
    head = loop.advance(1).tokens
    warm_out = loop.advance(warm)
    timed = loop.advance(args.steps)
    if timed.status != SmokeStatus.OK or timed.device_elapsed_ns == 0:
        print(json.dumps({"unavailable": f"reference session_advance failed: cuda_error {timed.cuda_error}"}))
        return
    session.destroy()
    rate = args.steps / (timed.device_elapsed_ns * 1e-9)
    tokens = head + warm_out.tokens + timed.tokens
    peaks = measured_peaks()
    nbytes = cfg.projection_bytes_per_token()
    print(json.dumps({
        "impl": "reference CUDA library (oracle/_ref/libnerva_ref_decode.so: the reference's session and kernels, "
                "cuBLASLt projections, built for sm_100)",
        "value": rate, "unit": UNIT, "steps": args.steps, "warmup": warm,
        "ms_per_step": 1e3 / rate, "graph_nodes": int(timed.graph_nodes),
        "whole_step_frac": nbytes * rate / 1e9 / peaks["hbm_gbs"],
        "setup_s": {"session_create_with_autotune": create_s, "prefill": prefill_s},
        "parity": parity_block(cfg, tokens),
    }), flush=True)


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
    timeline_steps = 8
    max_context = (cfg.prompt_tokens + 1 + args.warmup + 2 * args.steps + profile_steps + 2 * timeline_steps + 8 +
                   MAX_EXTRA_CLOCK_STEPS)
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
    clocks.mark()
    timed = loop.advance(args.steps)             # K graph replays, timed by CUDA events on the session stream
    sync()
    if timed.status != SmokeStatus.OK or len(timed.tokens) != args.steps:
        raise RuntimeError(f"timed advance failed: {timed.error}")
    device_s = timed.device_elapsed_ns * 1e-9
    # end to end: one C-ABI call per token, host clock, D2H of the slot + synchronise each step
    t0 = time.perf_counter()
    e2e_stream = []
    for _ in range(args.steps):
        out = loop.advance(1)
        e2e_stream += out.tokens
    e2e_s = time.perf_counter() - t0
    e2e_tokens = len(e2e_stream)
    # a timed region of a fraction of a second may end before the sampler has seen it: the same step keeps
    # running, untimed, until a few samples of the clocks under this load exist
    # (a number of steps every rank computes alike from the slowest rank's time: the ranks step together)
    agreed_s = _max_over_ranks(device_s, world)
    extra = extra_clock_steps(agreed_s, args.steps)
    if extra:
        loop.advance(extra)
    clock_info = clocks.stop()
    stream = first.tokens + warm.tokens + timed.tokens + e2e_stream

    # In-step time of every operator: a fork of the session (shared weights, cloned state) created
    # with the stamps switched on replays the same graph shape; the timed region above ran without them.
    busy = None
    if world == 1 and args.engine == 0:
        os.environ["NERVA_B200_TIMELINE"] = "1"
        fork = session.fork_shared_weights()
        if not args.timeline:
            del os.environ["NERVA_B200_TIMELINE"]
        if fork.status == SmokeStatus.OK:
            fork_loop = CudaHfDecodeSequenceLoop(fork)
            fork_loop.advance(3)
            busy = timeline_busy_us(fork, fork_loop, cfg, timeline_steps)
            fork.destroy()
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
    # parity on the oracle's history, position by position (restarts the session's request: last use of it)
    forced_parity = teacher_forced_parity(session, cfg) if world == 1 and args.engine == 0 else None
    session.destroy()

    device_s = _max_over_ranks(device_s, world)
    e2e_s = _max_over_ranks(e2e_s, world)
    proj_kinds = ("qkv", "o", "gate_up", "down", "lm_head")
    isolated_ns = sum(prof[k]["ns"] for k in proj_kinds) / profile_steps
    proj_launches = sum(prof[k]["launches_per_step"] for k in proj_kinds)
    # per GPU: this rank's weight slices + bf16 vectors
    bytes_per_token = ck.config.projection_bytes_per_token() + 2 * cfg.hidden * (3 * cfg.layers + 1)
    peaks = measured_peaks()
    step_us = 1e6 * device_s / args.steps
    kernel_name = "projection_stream_kernel (QKV, O, gate-up, down, lm_head)"
    if busy is not None:
        kernel_us = sum(busy[k] for k in proj_kinds)
        time_source = ("in-step: kernel-written %globaltimer stamps during ordinary graph replays of a fork of the "
                       "session, launches charged net of overlap with their predecessors")
    else:
        kernel_us = isolated_ns / 1e3
        time_source = "event-per-launch pass outside the graph (no in-step stamps on this configuration)"
    achieved = bytes_per_token / (kernel_us * 1e-6) / 1e9
    if args.engine == 1:
        # one kernel per token: its launch duration is the event-timed step itself; its
        # algorithmic bytes add the KV rows read at the mean timed context and the KV row written
        mean_ctx = cfg.prompt_tokens + 1 + max(args.warmup, 3) + args.steps / 2
        kv_bytes = cfg.layers * 2 * cfg.kv_hidden * 2 * (mean_ctx + 1)
        bytes_per_token = bytes_per_token + int(kv_bytes)
        proj_launches = 1
        kernel_name = "decode_step_kernel (whole step: projections + attention + sampling)"
        kernel_us = step_us
        time_source = "the event-timed step (one launch per token)"
        achieved = bytes_per_token / (device_s / args.steps) / 1e9
    value = args.steps / device_s  # all ranks decode the same sequence together
    result = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": 1000.0 * device_s / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_block(cfg, world),
        "timed_context": f"{cfg.prompt_tokens + 1 + max(args.warmup, 3)}.."
                         f"{cfg.prompt_tokens + 1 + max(args.warmup, 3) + args.steps}",
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
            "traffic_source": NCU_TRAFFIC_SOURCE,
            "launches_per_token": proj_launches, "bytes_per_token": bytes_per_token,
            "us_per_token": kernel_us, "time_source": time_source, "engine": args.engine,
            "isolated_frac": (bytes_per_token / (isolated_ns * 1e-9) / 1e9) / peaks["hbm_gbs"],
            "isolated_us_per_token": isolated_ns / 1e3,
            "whole_step_frac": (bytes_per_token * args.steps / device_s / 1e9) / peaks["hbm_gbs"],
        },
        "parity": dict(parity_block(cfg, stream), teacher_forced=forced_parity),
        "in_step_us_per_token": busy,
        "profile_us_per_token": {k: v["ns"] / profile_steps / 1e3 for k, v in prof.items()},
        "setup_s": {"generate_weights": gen_s, "session_create": create_s, "prefill": prefill_s},
        "graph_nodes": int(timed.graph_nodes),
        "token_hash": f"{timed.observed_token_hash:016x}",
    }
    if timeline is not None:
        result["timeline"] = timeline
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle as O
        rate, done, threads = cpu_decode_sample(ck, cfg, budget_s=float(os.environ.get("NERVA_CPU_BUDGET_S", "20")),
                                                max_tokens=8)
        result["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": threads, "kind": "port",
                                  "sample": cpu_sample_text(cfg, done, 8, threads)}
        del ck
        if not args.no_gpu_baseline:
            result["gpu_baseline"] = gpu_baseline_child(args, cfg)
    return result


def run_batch_workload(args, cfg) -> None:
    """32 forks of one session (shared weights, identical histories) advanced as packed blocks through
    nerva_cuda_hf_decode_sequence_batch_advance_one, against the same forks advanced one after the
    other with session_advance: the reference's shared-fork batch comparison
    (docs/source/perf/qwen3_8b_shared_fork_batch_compare_32req_target32.json)."""
    from nerva_b200 import build, ops, synth
    from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
    build.build()
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    steps, forks = args.steps, 32
    session = CudaHfDecodeSequenceSession(ck, cfg.prompt_tokens + 2 * steps + 16, use_descriptors=True)
    if session.status != SmokeStatus.OK:
        raise RuntimeError(f"session create failed: {session.error}")
    start, loop = CudaHfDecodeSequenceLoop.start(session, prompt)
    if start.status != SmokeStatus.OK:
        raise RuntimeError(f"session start failed: {start.error}")
    loop.advance(4)
    block = [session] + [session.fork_shared_weights() for _ in range(forks - 1)]
    lone = [session.fork_shared_weights() for _ in range(forks)]
    # warm-up: two block steps and two lone steps, with the logits of the first compared
    warm_block, warm_lone = [], []
    logit_gap = None
    for i in range(2):
        out = CudaHfDecodeSequenceSession.batch_advance_one(block, forks, forks)
        warm_block.append(out.tokens[0])
        warm_lone.append(CudaHfDecodeSequenceLoop(lone[0]).advance(1).tokens[0])
        if i == 0:
            a, b = block[0].read_logits(), lone[0].read_logits()
            top2 = np.sort(b)[-2:]
            logit_gap = {"max_abs_logit_difference": float(np.abs(a - b).max()),
                         "lone_top1_minus_top2": float(top2[1] - top2[0])}
    for s in lone[1:]:
        CudaHfDecodeSequenceLoop(s).advance(2)
    t0 = time.perf_counter()
    block_tokens = []
    for _ in range(steps):
        out = CudaHfDecodeSequenceSession.batch_advance_one(block, forks, forks)
        if out.status != SmokeStatus.OK or out.block_tokens != forks:
            raise RuntimeError(f"block step failed: reason {out.reason} {out.error}")
        block_tokens.append(out.tokens)
    block_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    lone_tokens = [CudaHfDecodeSequenceLoop(s).advance(steps).tokens for s in lone]
    lone_s = time.perf_counter() - t0
    same_within_block = all(len(set(row)) == 1 for row in block_tokens)
    stream = [row[0] for row in block_tokens]
    match = sum(1 for a, b in zip(stream, lone_tokens[0]) if a == b)
    first_diff = next((i for i, (a, b) in enumerate(zip(stream, lone_tokens[0])) if a != b), None)
    peaks = measured_peaks()
    nbytes = cfg.projection_bytes_per_token()
    print(json.dumps({
        "workload": "shared-fork batch: 32 sessions, one token each per block step", "config": config_block(cfg, 1),
        "block_tokens": forks, "steps": steps,
        "block_tok_s": forks * steps / block_s, "sequential_tok_s": forks * steps / lone_s,
        "speedup": lone_s / block_s, "ms_per_block_step": 1e3 * block_s / steps,
        "weight_stream_frac_of_measured_hbm": nbytes / (block_s / steps) / 1e9 / peaks["hbm_gbs"],
        "tokens_identical_within_block": same_within_block,
        "token_match_with_sequential": {"compared": steps, "identical_prefix": steps if first_diff is None else first_diff,
                                        "warm_up_block_tokens": warm_block, "warm_up_lone_tokens": warm_lone,
                                        "first_step": logit_gap},
        "timing": "host wall clock around the C-ABI calls, token slots copied back every call",
    }), flush=True)


def run_deepseek_workload(args, rank: int = 0, world: int = 1) -> None:
    """DeepSeek-V2-Lite architecture (latent attention + softmax top-6 of 64 experts + always-on shared
    experts, dense first layer): batch-1 greedy decode after a 1024-token prompt, on one GPU or
    expert-parallel over `world` GPUs (every rank holds 64 / world routed experts and 1 / world of the
    shared expert of each sparse layer, everything else whole).  The bytes a token must stream are the
    matrices it touches (attention projections, router, 6 routed + the shared expert matrices per sparse
    layer, lm_head), not the 31 GB that are resident."""
    import dataclasses
    from nerva_b200 import build, ops, synth
    from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
    build.build()
    cfg = synth.DEEPSEEK_V2_LITE
    if args.layers:
        cfg = dataclasses.replace(cfg, layers=args.layers, name=f"{cfg.name} cut to {args.layers} layers")
    if args.prompt_tokens:
        cfg = dataclasses.replace(cfg, prompt_tokens=args.prompt_tokens)
    max_context = cfg.prompt_tokens + max(args.warmup, 3) + 2 * args.steps + 16 + MAX_EXTRA_CLOCK_STEPS
    t0 = time.perf_counter()
    if world > 1:
        from nerva_b200 import tp
        t1 = t0
        session = tp.create_session(cfg, max_context, rank, world)  # generates this rank's part and connects the ranks
    else:
        ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
        t1 = time.perf_counter()
        session = CudaHfDecodeSequenceSession(ck, max_context)
    if session.status != SmokeStatus.OK:
        raise RuntimeError(f"session create failed: {session.error}")
    t2 = time.perf_counter()
    start, loop = CudaHfDecodeSequenceLoop.start(session, synth.prompt_ids(cfg))
    if start.status != SmokeStatus.OK:
        raise RuntimeError(f"session start failed: {start.error}")
    t3 = time.perf_counter()
    loop.advance(max(args.warmup, 3))
    sync = _barrier_fn(world)
    sampler = ClockSampler(int(os.environ.get("NERVA_GPU_INDEX", "0")))
    sampler.start()
    sync()
    sampler.mark()
    timed = loop.advance(args.steps)
    sync()
    if timed.status != SmokeStatus.OK or len(timed.tokens) != args.steps:
        raise RuntimeError(f"timed advance failed: {timed.error}")
    device_s = _max_over_ranks(timed.device_elapsed_ns * 1e-9, world)
    t4 = time.perf_counter()
    e2e_tokens = []
    for _ in range(args.steps):
        out = loop.advance(1)
        if out.status != SmokeStatus.OK:
            raise RuntimeError(f"advance failed: {out.error}")
        e2e_tokens += out.tokens
    e2e_s = _max_over_ranks(time.perf_counter() - t4, world)
    extra = extra_clock_steps(device_s, args.steps)  # as in the dense bench: a few clock samples under this load
    if extra:
        loop.advance(extra)
    clocks = sampler.stop()
    # where the step's time goes: events between launch groups, un-captured (includes event overhead)
    profile_us = None
    if world == 1:
        profile = session.profile_steps(4)
        profile_us = {name: entry["ns"] / 4 / 1e3 for name, entry in profile.items()}
    peaks = measured_peaks()
    nbytes = cfg.active_weight_bytes_per_token()
    r = session.create_result
    sync()
    if rank != 0:
        session.destroy()
        return
    print(json.dumps({
        "metric": "DeepSeek-V2-Lite-arch BF16 batch-1 decode tok/s", "value": args.steps / device_s, "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": 1e3 * device_s / args.steps,
        "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{cfg.name}: {cfg.layers} layers, hidden {cfg.hidden}, {cfg.heads} heads, latent rank "
                               f"{cfg.kv_lora_rank}, nope {cfg.qk_nope_head_dim} / rope {cfg.qk_rope_head_dim} / v "
                               f"{cfg.head_dim}; {cfg.dense_layers} dense layer (intermediate {cfg.intermediate}), then "
                               f"{cfg.num_experts} experts top-{cfg.top_k} softmax + shared {cfg.shared_intermediate}, "
                               f"expert intermediate {cfg.moe_intermediate}; vocab {cfg.vocab}; batch 1, "
                               f"{cfg.prompt_tokens}-token seeded prompt, greedy decode",
                   "weights": "random-init bf16 ~N(0,0.02) seed 0, unit norm weights (synthetic)",
                   "parallelism": "single GPU" if world == 1 else
                                  f"ep{world}: routed experts and the shared expert's intermediate divided over the ranks, "
                                  f"everything else whole on every rank; partial MLP outputs exchanged over NVLink peer memory",
                   "active_weight_bytes_per_token": nbytes, "resident_weight_bytes": int(r.resident_weight_bytes),
                   "resident_kv_bytes": int(r.resident_kv_bytes)},
        "clocks": clocks,
        "e2e": {"value": args.steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 44},
        "roofline": {"bound": "hbm", "kernel": "whole step (projection, latent attention and expert stream kernels)",
                     "achieved": nbytes / device_s * args.steps / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": nbytes / device_s * args.steps / 1e9 / peaks["hbm_gbs"], "peak_source": peaks["source"],
                     "traffic": None},
        "token_hash": f"{timed.observed_token_hash:016x}",
        "profile_us_per_token": profile_us,
        "profile_note": "event-per-launch pass outside the graph: qkv = first projection, attention = the three "
                        "latent-attention kernels, o = output projection, gate_up = dense gate/up, down = dense down "
                        "or the two expert-stream kernels (routing + gate/up, down)",
        "setup_s": {"generate_weights": t1 - t0, "session_create": t2 - t1, "prefill": t3 - t2},
    }), flush=True)
    session.destroy()


def run_operator_workloads(kind: str, only_shape: str = "", only_tokens: int = 0, only_batch: int = 0,
                           only_context: int = 0) -> None:
    """Per-operator sweeps (isolated projection shapes, long-context attention) through the per-op C ABI (host buffers in,
    device time per launch out, L2 flushed between launches).  One JSON line per case."""
    from nerva_b200 import build, ops, synth
    build.build()
    peak = measured_peaks()
    if kind == "linear":
        shapes = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288),
                  ("lm_head", 151936, 4096)]
        for name, rows, cols in shapes:
            if only_shape and name != only_shape:
                continue
            w = ops.synth_normal_bf16(0, 77, rows * cols, 0.02)
            for m in (1, 4, 16, 64):
                if only_tokens and m != only_tokens:
                    continue
                x = ops.synth_normal_bf16(0, synth.T_ACTIVATION, m * cols, 1.0)
                _, alone_ns = ops.projection(w, x, rows, cols, tokens=m, warmup=3, iterations=10)
                # sustained: copies of the matrix that together exceed the 126 MB L2, launched back to back
                copies = max(2, -(-320_000_000 // (2 * rows * cols)))
                y, ns = ops.projection_sustained(w, x, rows, cols, tokens=m, copies=copies, warmup=2 * copies,
                                                 iterations=8 * copies)
                nbytes = 2 * rows * cols + 2 * m * cols + 4 * m * rows
                gbs = nbytes / ns
                print(json.dumps({"workload": "decode-linear", "shape": name, "N": rows, "K": cols, "M": m,
                                  "us": ns / 1e3, "algorithmic_bytes": nbytes, "GB/s": gbs,
                                  "frac_of_measured_hbm": gbs / peak["hbm_gbs"],
                                  "timing": f"{8 * copies} launches back to back over {copies} copies of the matrix "
                                            f"(larger than L2 together), programmatic dependent launch",
                                  "single_launch_us": alone_ns / 1e3,
                                  "single_launch_frac": nbytes / alone_ns / peak["hbm_gbs"],
                                  "note": "block kernel on the tensor pipe (tcgen05), weights streamed once for the block"
                                  if m > 1 else "weight-streaming GEMV"}), flush=True)
        return
    run_attention_workload(1, 0, only_batch, only_context)


def run_attention_workload(world: int, rank: int, only_batch: int = 0, only_context: int = 0,
                           emulated: bool = False) -> None:
    """Long-context GQA decode attention on the Qwen3-8B layer shape (32 query / 8 KV heads of 128),
    bf16 K/V in 16-token pages placed by a seeded permutation.  With world > 1 the KV heads are
    sharded the way the tensor-parallel session shards them: every rank owns 8 / world KV heads
    (their pages and page table) and the 32 / world query heads that read them.  Attention needs
    no exchange, and none follows it: a rank's output slice is exactly the input columns of its
    shard of the O projection.  The time of a case is the slowest rank's."""
    from nerva_b200 import build, ops, synth
    build.build()
    peak = measured_peaks()
    heads, kv_heads, d = 32 // world, 8 // world, 128
    for batch in (1, 8):
        for context in (8192, 32768, 131072):
            if (only_batch and batch != only_batch) or (only_context and context != only_context):
                continue
            pages = (context + 15) // 16
            n = batch * pages * 16 * kv_heads * d
            k = ops.synth_normal_bf16(rank, synth.layer_tensor_id(0, synth.L_K), n, 1.0)
            v = ops.synth_normal_bf16(rank, synth.layer_tensor_id(0, synth.L_V), n, 1.0)
            table = np.stack([synth.permutation(b, synth.T_PAGE_TABLE, pages) for b in range(batch)])
            q = synth.normal_f32(rank, synth.layer_tensor_id(0, synth.L_Q), batch * heads * d, 1.0)
            _, alone_ns = ops.gqa_decode_attention(q, k, v, table, batch, context, heads, kv_heads, d, warmup=3,
                                                   iterations=10)
            # sustained: the caches of several layers (together larger than the L2), one launch after the other
            copies = max(2, min(36, -(-320_000_000 // (4 * n))))
            out, ns = ops.gqa_decode_attention_sustained(q, k, v, table, batch, context, heads, kv_heads, d,
                                                         copies=copies, warmup=copies, iterations=4 * copies)
            # emulated: one rank's shard measured alone on this GPU (every rank does the same work)
            total_ns = float(ns) if emulated else _max_over_ranks(float(ns), world)
            # whole job: all KV heads of all ranks
            nbytes = world * batch * (2 * context * kv_heads * d * 2 + pages * 4 + heads * d * 4 * 2)
            gbs = nbytes / total_ns
            if rank == 0:
                print(json.dumps({"workload": "long-context GQA decode attention", "n_gpus": world, "batch": batch,
                                  "context": context, "heads": 32, "kv_heads": 8, "head_dim": d,
                                  "us": total_ns / 1e3, "algorithmic_bytes": nbytes,
                                  "GB/s": gbs, "frac_of_measured_hbm_per_gpu": gbs / world / peak["hbm_gbs"],
                                  "sharding": "none" if world == 1 else f"{kv_heads} KV heads per rank, no exchange "
                                                                         f"(slowest rank's time)",
                                  "pages": "16-token pages placed by a seeded Fisher-Yates permutation",
                                  "timing": f"{4 * copies} launches back to back over the caches of {copies} layers "
                                            f"(larger than L2 together)",
                                  "single_launch_us": (float(alone_ns) if emulated else
                                                       _max_over_ranks(float(alone_ns), world)) / 1e3,
                                  "ranks_measured": "one rank's shard on one GPU" if emulated else "all",
                                  "single_launch_note": "one launch timed alone, 192 MB written to flush L2 before it"}),
                      flush=True)


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
    ap.add_argument("--no-gpu-baseline", action="store_true",
                    help="skip the child process that times the reference's own CUDA library on this workload")
    ap.add_argument("--engine", type=int, default=0, choices=[0, 1],
                    help="0: one kernel per operator in a CUDA graph; 1: the whole-step kernel")
    ap.add_argument("--layers", type=int, default=0,
                    help="cut the model to this many layers (profiler captures only; not a bench line)")
    ap.add_argument("--prompt-tokens", type=int, default=0, help="override the prompt length")
    ap.add_argument("--workload", default="decode", choices=["decode", "linear", "attention", "reference-gpu", "batch", "deepseek"],
                    help="decode: the bench line; linear / attention: per-operator sweeps of the isolated "
                         "projection shapes and of long-context attention (one JSON line per case)")
    ap.add_argument("--shape", default="", help="linear sweep: only this projection (qkv, o, gate_up, down, lm_head)")
    ap.add_argument("--tokens", type=int, default=0, help="linear sweep: only this block size")
    ap.add_argument("--batch", type=int, default=0, help="attention sweep: only this batch size")
    ap.add_argument("--context", type=int, default=0, help="attention sweep: only this context length")
    ap.add_argument("--shard-of", type=int, default=0, choices=[0, 2, 4, 8],
                    help="attention sweep on one GPU: measure one rank's shard of an N-way split by KV head")
    ap.add_argument("--timeline", action="store_true",
                    help="add the in-graph timeline (kernel-written %%globaltimer stamps, mean over layers)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "attention" and world > 1:
        visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        from nerva_b200 import tp
        tp.select_device(local)
        import torch.distributed as dist
        dist.init_process_group("gloo")  # carries the host-side max over ranks only
        run_attention_workload(world, rank, args.batch, args.context)
        dist.barrier()
        dist.destroy_process_group()
        return
    if args.workload == "attention" and args.shard_of and world == 1:
        run_attention_workload(args.shard_of, 0, args.batch, args.context, emulated=True)
        return
    if args.workload in ("linear", "attention"):
        if rank == 0:
            run_operator_workloads(args.workload, args.shape, args.tokens, args.batch, args.context)
        return
    cfg = workload(args.config, args.layers, args.prompt_tokens)
    if args.workload == "reference-gpu":
        if rank == 0:
            run_reference_gpu(args, cfg)
        return
    if args.workload == "batch":
        if rank == 0:
            run_batch_workload(args, cfg)
        return
    if args.workload == "deepseek":
        if world > 1:
            from nerva_b200 import tp
            tp.select_device(local)
            os.environ["NERVA_GPU_INDEX"] = str(local)
            import torch.distributed as dist
            dist.init_process_group("gloo")
            run_deepseek_workload(args, rank, world)
            dist.barrier()
            dist.destroy_process_group()
        else:
            run_deepseek_workload(args)
        return
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
