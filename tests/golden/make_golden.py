"""Regenerates the committed fixtures under tests/golden/.

    python tests/golden/make_golden.py

1. tiny_qwen3.json — the CPU oracle (both numeric contracts) on the tiny
   Qwen3-architecture configuration: 64-token seeded prompt, 32 greedy tokens,
   plus a sample of logits per step.  The oracle itself is pinned by the
   reference's known-answer tests (tests/test_cpu_oracle.py).
2. abi_layout.txt — sizeof/offsetof of every ABI struct, measured by compiling
   a probe against the REFERENCE header (needs the reference checkout, only
   present on the build machine).  The test-suite compares this library's
   header against it.
3. abi_prototypes.txt — return and parameter types, in order, of every
   nerva_cuda_* function this library declares, as the REFERENCE header
   declares them.
4. qwen3_8b.json (only with the argument `qwen3_8b`; takes about an hour and 20 GB on 8 cores) —
   the CPU oracle on the full 36-layer Qwen3-8B-architecture model with the 512-token seeded
   prompt: per decoded position the token, the top-1 minus top-2 margin, the largest logit, the
   top-8 candidates and 64 sampled logits (CUDA contract: 64 positions; CPU contract: 32), and a
   depth sweep (models cut to 1, 2, 4, 8, 16, 36 layers, 16-token prompt): 1024 sampled logits
   under the serial summation order, and the oracle's distance to itself when only the
   summation order changes (8 interleaved partial sums).
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
sys.path.insert(0, ROOT)

from nerva_b200 import ffi, synth  # noqa: E402
from oracle import oracle as O  # noqa: E402

REFERENCE_HEADER = os.path.join(O.REFERENCE_ROOT, "native/cuda/nerva_cuda_api.h")
SAMPLE_INDICES = [0, 1, 2, 3, 101, 1009, 4099, 8191, 12345, 16000, 20011, 25000, 29999, 31000, 31998, 31999]


def tiny_golden() -> dict:
    cfg = synth.TINY_QWEN3
    ck = synth.dense_checkpoint(cfg)
    prompt = synth.prompt_ids(cfg)
    out = {"config": cfg.name, "prompt": prompt.tolist(), "sample_indices": SAMPLE_INDICES}
    for name, mode in (("cpu", O.MODE_CPU), ("cuda", O.MODE_CUDA)):
        dec = O.Decoder(ck, cfg.prompt_tokens + cfg.decode_tokens, mode=mode)
        tokens, logits = dec.decode_greedy(prompt, cfg.decode_tokens, want_logits=True)
        top2 = np.sort(logits, axis=1)[:, -2:]
        out[name] = {
            "tokens": tokens.tolist(),
            "token_hash": O.hash_tokens(tokens),
            "logit_samples": [[float(v) for v in row[SAMPLE_INDICES]] for row in logits],
            "top1_minus_top2": [float(b - a) for a, b in top2],
            "max_logit": [float(v) for v in logits.max(axis=1)],
        }
    return out


QWEN_SAMPLE_INDICES = [int(i) for i in np.linspace(0, 151935, 64).astype(np.int64)]
SWEEP_DEPTHS = [1, 2, 4, 8, 16, 36]
SWEEP_PROMPT_TOKENS = 16
SWEEP_SAMPLE_INDICES = [int(i) for i in np.linspace(0, 151935, 1024).astype(np.int64)]


def _prefix_checkpoint(full, layers: int):
    """The first `layers` layers of `full` as a checkpoint of its own (same tensors, no copy)."""
    import dataclasses
    cfg = dataclasses.replace(full.config, name=f"{full.config.name}-cut{layers}", layers=layers)
    return synth.DenseCheckpoint(cfg, full.embeddings, full.final_norm, full.lm_head, full.layers[:layers])


def _record_stream(dec, prompt, steps: int, log) -> dict:
    """Greedy decode step by step, keeping per position what the GPU test compares against."""
    out = {"tokens": [], "top1_minus_top2": [], "max_logit": [], "logit_samples": [], "top8_index": [],
           "top8_value": []}
    for i, token in enumerate(prompt[:-1]):
        dec.step(int(token), want_logits=False)
        if i % 64 == 0:
            log(f"  prompt {i}/{len(prompt)}")
    current = int(prompt[-1])
    for step in range(steps):
        logits = dec.step(current, want_logits=True)
        order = np.argsort(-logits, kind="stable")[:8]
        current = O.argmax(logits, dec.mode if dec.mode != O.MODE_CPU else O.MODE_CUDA)
        out["tokens"].append(int(current))
        out["top1_minus_top2"].append(float(logits[order[0]] - logits[order[1]]))
        out["max_logit"].append(float(logits[order[0]]))
        out["logit_samples"].append([float(v) for v in logits[QWEN_SAMPLE_INDICES]])
        out["top8_index"].append([int(v) for v in order])
        out["top8_value"].append([float(v) for v in logits[order]])
        log(f"  token {step}: {current} margin {out['top1_minus_top2'][-1]:.4f}")
    out["token_hash"] = O.hash_tokens(out["tokens"])
    return out


def qwen3_8b_golden(threads: int = 0) -> dict:
    import time
    t0 = time.time()

    def log(text):
        print(f"[{time.time() - t0:7.0f}s] {text}", flush=True)

    if threads:
        O.lib().oracle_set_threads(threads)
    cfg = synth.QWEN3_8B
    log("generating the checkpoint")
    ck = synth.dense_checkpoint(cfg, fill=O.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    out = {"config": cfg.name, "prompt_tokens": int(prompt.size), "prompt_hash": O.hash_tokens(prompt),
           "sample_indices": QWEN_SAMPLE_INDICES}
    # depth sweep first: it is the cheap part
    sweep_prompt = synth.prompt_ids(cfg, count=SWEEP_PROMPT_TOKENS)
    sweep = {"depths": SWEEP_DEPTHS, "prompt_tokens": SWEEP_PROMPT_TOKENS, "sample_indices": SWEEP_SAMPLE_INDICES,
             "serial_samples": [], "lanes8_samples": [], "self_distance": [], "serial_argmax": [],
             "serial_margin": []}
    for depth in SWEEP_DEPTHS:
        cut = _prefix_checkpoint(ck, depth)
        rows = []
        for lanes in (1, 8):
            O.set_sum_lanes(lanes)
            dec = O.Decoder(cut, SWEEP_PROMPT_TOKENS, mode=O.MODE_CUDA)
            for token in sweep_prompt[:-1]:
                dec.step(int(token), want_logits=False)
            rows.append(dec.step(int(sweep_prompt[-1]), want_logits=True))
            dec.close()
        O.set_sum_lanes(1)
        top2 = np.sort(rows[0])[-2:]
        sweep["serial_samples"].append([float(v) for v in rows[0][SWEEP_SAMPLE_INDICES]])
        sweep["lanes8_samples"].append([float(v) for v in rows[1][SWEEP_SAMPLE_INDICES]])
        sweep["self_distance"].append(float(np.abs(rows[0] - rows[1]).max()))
        sweep["serial_argmax"].append(int(np.argmax(rows[0])))
        sweep["serial_margin"].append(float(top2[1] - top2[0]))
        log(f"depth {depth}: oracle self-distance {sweep['self_distance'][-1]:.4e}")
    out["depth_sweep"] = sweep
    for name, mode, steps in (("cuda", O.MODE_CUDA, 64), ("cpu", O.MODE_CPU, 32)):
        log(f"contract {name}: {prompt.size}-token prompt, {steps} greedy tokens")
        dec = O.Decoder(ck, cfg.prompt_tokens + steps, mode=mode)
        out[name] = _record_stream(dec, prompt, steps, log)
        dec.close()
    return out


def layout_probe_source(header: str) -> str:
    lines = ["#include <stddef.h>", "#include <stdio.h>", f'#include "{header}"', "int main(void) {"]
    for name, cls in ffi.structs.items():
        if not name.startswith("NervaCuda"):
            continue  # additive structs of this library have no counterpart in the reference header
        lines.append(f'  printf("{name} %zu\\n", sizeof({name}));')
        for fname, _ in cls._fields_:
            lines.append(f'  printf("{name}.{fname} %zu\\n", offsetof({name}, {fname}));')
    lines += ["  return 0;", "}"]
    return "\n".join(lines)


def measure_layout(header: str) -> str:
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "probe.c")
        exe = os.path.join(tmp, "probe")
        with open(src, "w") as f:
            f.write(layout_probe_source(header))
        subprocess.run(["gcc", "-o", exe, src], check=True)
        return subprocess.run([exe], check=True, capture_output=True, text=True).stdout


def prototypes(header_text: str, prefix: str = "nerva_cuda_") -> dict:
    """name -> 'return_type(param_type, ...)' with parameter names and comments removed."""
    import re
    text = re.sub(r"/\*.*?\*/", "", header_text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    found = {}
    for m in re.finditer(r"([A-Za-z_][\w \*]*?)\b(" + prefix + r"\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, params = m.group(1), m.group(2), m.group(3)
        types = []
        for p in params.split(","):
            p = " ".join(p.split())
            p = re.sub(r"\b\w+$", "", p).strip() if p != "void" else p   # drop the parameter name
            types.append(re.sub(r"\s*\*\s*", "*", p))
        found[name] = f"{' '.join(ret.split())}({', '.join(types)})"
    return found


def reference_prototypes() -> str:
    """Prototypes, as the reference header declares them, of every nerva_cuda_* function that
    this repository's header declares."""
    with open(REFERENCE_HEADER) as f:
        ref = prototypes(f.read())
    with open(ffi.HEADER) as f:
        ours = prototypes(f.read())
    return "".join(f"{name} {ref[name]}\n" for name in sorted(ours))


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "qwen3_8b":
        golden = qwen3_8b_golden(int(sys.argv[2]) if len(sys.argv) > 2 else 0)
        with open(os.path.join(HERE, "qwen3_8b.json"), "w") as f:
            json.dump(golden, f, indent=None, separators=(",", ":"))
        sys.exit(0)
    with open(os.path.join(HERE, "tiny_qwen3.json"), "w") as f:
        json.dump(tiny_golden(), f, indent=1)
    if os.path.exists(REFERENCE_HEADER):
        with open(os.path.join(HERE, "abi_layout.txt"), "w") as f:
            f.write(measure_layout(REFERENCE_HEADER))
        with open(os.path.join(HERE, "abi_prototypes.txt"), "w") as f:
            f.write(reference_prototypes())
    else:
        print("reference header not present: abi_layout.txt left untouched")
