"""The command line, in the manner of the reference's engine binary (engine/src/main.c:38-141, 211-303).

    vitna-anchor generate --model <dir> (--ids a,b,... | --ids-file f) [--max-new n] [--greedy |
                 --temperature t [--top-k k] [--top-p p] [--seed s]] [--logits-out file] [--timing]
                 [--ctx n] [--parallel n] [--stop-at-special] [--device cuda] [--dtype bfloat16|float32]
                 [--kv-block n] [--num-pages n] [--max-batch-tokens n] [--max-prompt-portion n]
    vitna-anchor logits   --model <dir> (--ids ... | --ids-file f) --out file [--ctx n] [--dtype ...]
    vitna-anchor random-model --config file.json --seed s --out <dir> [--std x] [--norm-noise x] [--weights-dtype ...]
    vitna-anchor info     --model <dir>

generate prints JSON {"prompt_ids": [...], "ids": [...]} (main.c:1118-1124; there is no tokenizer
here, so no text).  logits writes every prompt position's logits as float32, little-endian,
positions x vocab (main.c:900-937).  An unknown option is an error and the exit code is 1
(main.c:296-299).
"""
from __future__ import annotations

import json
import sys
from typing import List, Optional

VALUE_OPTIONS = {"--model", "--ids", "--ids-file", "--max-new", "--temperature", "--top-k", "--top-p", "--seed", "--logits-out",
                 "--out", "--ctx", "--device", "--dtype", "--parallel", "--kv-block", "--num-pages", "--max-batch-tokens",
                 "--max-prompt-portion", "--config", "--std", "--norm-noise", "--weights-dtype"}
FLAG_OPTIONS = {"--greedy", "--timing", "--stop-at-special"}
COMMANDS = ("generate", "logits", "random-model", "info")


class UsageError(Exception):
    pass


def parse_args(argv: List[str]) -> dict:
    a = {"max_new": 64, "temperature": 0.0, "top_k": 0, "top_p": 1.0, "seed": 0, "device": "cuda", "dtype": "bfloat16"}
    i = 0
    while i < len(argv):
        k = argv[i]
        if k in FLAG_OPTIONS:
            if k == "--greedy":
                a["temperature"] = 0.0
            else:
                a[k[2:].replace("-", "_")] = True
            i += 1
        elif k in VALUE_OPTIONS and i + 1 < len(argv):
            a[k[2:].replace("-", "_")] = argv[i + 1]
            i += 2
        else:
            raise UsageError(f"Unknown or incomplete option: {k}")
    try:
        for key in ("max_new", "top_k", "seed", "ctx", "parallel", "kv_block", "num_pages", "max_batch_tokens", "max_prompt_portion"):
            if key in a:
                a[key] = int(a[key])
        for key in ("temperature", "top_p", "std", "norm_noise"):
            if key in a:
                a[key] = float(a[key])
    except ValueError as e:
        raise UsageError(f"a number was expected: {e}") from None
    return a


def read_ids(a: dict) -> List[int]:
    text = a.get("ids")
    if "ids_file" in a:
        try:
            with open(a["ids_file"], "r", encoding="utf-8") as f:
                text = f.read()
        except OSError as e:
            raise UsageError(f"cannot read {a['ids_file']}: {e.strerror}") from None
    if text is None:
        raise UsageError("give the prompt as --ids a,b,... or --ids-file <file> (this engine has no tokenizer)")
    try:
        ids = [int(t) for t in text.replace("\n", ",").split(",") if t.strip()]
    except ValueError:
        raise UsageError("--ids takes token ids separated by commas") from None
    if not ids:
        raise UsageError("the prompt is empty")
    return ids


def make_engine(a: dict):
    from ..engine.engine import Engine
    if "model" not in a:
        raise UsageError("--model <dir> is needed")
    if a["device"] not in ("cuda",):
        raise UsageError(f"--device is cuda; this engine has no path for {a['device']}")
    kw = {}
    for key, name in (("ctx", "ctx"), ("parallel", "parallel"), ("kv_block", "kv_block"), ("num_pages", "num_pages"),
                      ("max_batch_tokens", "max_batch_tokens"), ("max_prompt_portion", "max_prompt_portion")):
        if key in a:
            kw[name] = a[key]
    kw.setdefault("parallel", 1)
    return Engine(a["model"], dtype=a["dtype"], device=a["device"], **kw)


def cmd_generate(a: dict) -> int:
    ids = read_ids(a)
    eng = make_engine(a)
    stop = set()
    if a.get("stop_at_special") and getattr(eng.model.config, "eos_token_id", None) is not None:
        stop.add(eng.model.config.eos_token_id)
    out = eng.generate(ids, max_new=a["max_new"], temperature=a["temperature"], top_k=a["top_k"], top_p=a["top_p"],
                       seed=a["seed"], stop_ids=stop, logits_out=a.get("logits_out"))
    print(json.dumps({"prompt_ids": ids, "ids": out}))
    if a.get("timing"):
        t = eng.last_timing
        each = t["decode_ms"] / t["tokens_after_first"] if t["tokens_after_first"] else 0.0
        print(f"timing: {t['prompt_tokens']} prompt tokens in {t['prompt_ms']:.1f} ms; {t['tokens_after_first']} tokens after the "
              f"first new one in {t['decode_ms']:.1f} ms, {each:.2f} ms each", file=sys.stderr)
    return 0


def cmd_logits(a: dict) -> int:
    import numpy as np
    ids = read_ids(a)
    if "out" not in a:
        raise UsageError("logits needs --out <file>")
    eng = make_engine(a)
    rows = eng.logits(ids)
    np.ascontiguousarray(rows.cpu().numpy(), dtype="<f4").tofile(a["out"])
    print(json.dumps({"positions": len(ids), "vocab": int(rows.shape[1]), "out": a["out"]}))
    return 0


def cmd_random_model(a: dict) -> int:
    import torch
    from ..engine.loading import write_random_model
    for key in ("config", "out"):
        if key not in a:
            raise UsageError(f"random-model needs --{key}")
    with open(a["config"], "r", encoding="utf-8") as f:
        cfg = json.load(f)
    wd = {"bfloat16": torch.bfloat16, "float32": torch.float32}.get(a.get("weights_dtype", "bfloat16"))
    if wd is None:
        raise UsageError("--weights-dtype is bfloat16 or float32")
    write_random_model(a["out"], cfg, a["seed"], std=a.get("std", 0.02), norm_noise=a.get("norm_noise", 0.0), matrix_dtype=wd)
    print(json.dumps({"model": a["out"], "seed": a["seed"]}))
    return 0


def cmd_info(a: dict) -> int:
    from ..config import read_config_json, resolve
    if "model" not in a:
        raise UsageError("--model <dir> is needed")
    cj = read_config_json(a["model"])
    arch = resolve(cj)
    cfg = arch.parse_config(cj)
    print(json.dumps({"architecture": arch.name, "config": cfg.to_dict() if hasattr(cfg, "to_dict") else cj}))
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(__doc__)
        return 0 if argv else 1
    cmd, rest = argv[0], argv[1:]
    if cmd not in COMMANDS:
        print(f"Unknown command: {cmd}\n{__doc__}", file=sys.stderr)
        return 1
    try:
        a = parse_args(rest)
        return {"generate": cmd_generate, "logits": cmd_logits, "random-model": cmd_random_model, "info": cmd_info}[cmd](a)
    except UsageError as e:
        print(str(e), file=sys.stderr)
        return 1
    except Exception as e:   # refusals of the model, the checkpoint or the request: say why and stop
        print(f"{type(e).__name__}: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
