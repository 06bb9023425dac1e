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

REFERENCE_HEADER = os.path.join(os.environ.get("NERVA_REFERENCE_ROOT", "/root/reference"), "native/cuda/nerva_cuda_api.h")
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
    with open(os.path.join(HERE, "tiny_qwen3.json"), "w") as f:
        json.dump(tiny_golden(), f, indent=1)
    if os.path.exists(REFERENCE_HEADER):
        with open(os.path.join(HERE, "abi_layout.txt"), "w") as f:
            f.write(measure_layout(REFERENCE_HEADER))
        with open(os.path.join(HERE, "abi_prototypes.txt"), "w") as f:
            f.write(reference_prototypes())
    else:
        print("reference header not present: abi_layout.txt left untouched")
