#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ with the reference's own CPU program.

Usage: python tests/golden/make_golden.py /path/to/reference

It compiles the reference engine for the CPU (gcc, no CUDA), writes the two tiny
random models of tests/tiny_configs.py with this framework's random-weights
mode, and runs the reference's `logits --model DIR --ids ... --out FILE` on
them (engine/src/main.c:900-937): float32 logits [positions, vocab] computed
by engine/src/model.c, token by token.  The outputs are a few KB and are
committed; test_plain.py regenerates the same model folders from their seeds
and checks the plain implementation against these files.
"""
import glob
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tiny_configs import TINIES, write_tiny  # noqa: E402

IDS = {
    "tinyA": [5, 17, 33, 100, 255, 0, 7, 7, 7, 31, 2, 200, 64, 128, 1, 99, 45, 180, 12, 250, 3],
    "tinyB": [1, 9, 40, 100, 383, 0, 7, 7, 7, 301, 222, 57, 8, 350, 19, 76, 5, 5, 123],
}


def main(reference: str) -> None:
    work = tempfile.mkdtemp(prefix="golden_")
    exe = os.path.join(work, "reference-engine")
    srcs = sorted(glob.glob(os.path.join(reference, "engine", "src", "*.c")))
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-I", os.path.join(reference, "engine", "include"), *srcs,
                    "-lm", "-lpthread", "-o", exe], check=True)
    meta = {}
    for name, tiny in TINIES.items():
        mdir = write_tiny(os.path.join(work, name), tiny)
        out = os.path.join(HERE, f"{name}_logits.f32")
        subprocess.run([exe, "logits", "--model", mdir, "--ids", ",".join(map(str, IDS[name])), "--out", out], check=True)
        meta[name] = {"ids": IDS[name], "vocab": tiny["config"]["vocab_size"], "file": os.path.basename(out)}
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print("wrote", meta)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
