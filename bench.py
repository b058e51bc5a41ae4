#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

The default run is SmolLM2-135M's sizes with random weights (N(0, 0.02), norm weights 1, seed 0) in
bfloat16, a batch of 8 requests each decoding from its own 2,048-token random prompt, cache context
4,096, pages of 16.  A "step" is one decode step of the whole batch.

  value     decoded tokens a second through the step function (CUDA events around K steps)
  e2e       the same through the Python entry point (Engine.step: host token ids in, host token ids out)
  prefill   one 2,048-token prompt in one step: tokens a second, and flops / time / peak
  roofline  bytes the decode step must read (every weight once, the live requests' cache) / its time / peak
  points    decoded tokens a second at batch 1 and 64

Every step reads more than the 126 MB of L2 (weights 269 MB alone), so no flush is needed between
timed iterations.  Peaks come from MEASURED_PEAKS.json when the driver wrote it, else the pool's
earlier measurement (6.65 TB/s, 1.59 PFLOP/s bf16).
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2..4]: SmolLM2-135M (the default), 360M and 1.7B
MODELS = {
    "135M": dict(num_hidden_layers=30, hidden_size=576, intermediate_size=1536, num_attention_heads=9, num_key_value_heads=3,
                 head_dim=64, vocab_size=49152, max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=100000.0,
                 tie_word_embeddings=True),
    "360M": dict(num_hidden_layers=32, hidden_size=960, intermediate_size=2560, num_attention_heads=15, num_key_value_heads=5,
                 head_dim=64, vocab_size=49152, max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=100000.0,
                 tie_word_embeddings=True),
    "1.7B": dict(num_hidden_layers=24, hidden_size=2048, intermediate_size=8192, num_attention_heads=32, num_key_value_heads=32,
                 head_dim=64, vocab_size=49152, max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=130000.0,
                 tie_word_embeddings=True),
}
MODEL_NAME = "135M"
SIZES = dict(MODELS[MODEL_NAME])
PROMPT_LEN, CONTEXT, KV_BLOCK, PREFILL_TOKENS = 2048, 4096, 16, 2048
PROFILE_REGION = ""     # "decode" or "prefill": that timed region is bracketed by cudaProfilerStart/Stop (ncu --profile-from-start off)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(path) as f:
            m = json.load(f)
        if m.get("hbm_gbs"):
            out["hbm_gbs"] = float(m["hbm_gbs"])
        if m.get("bf16_tflops"):
            out["bf16_tflops"] = float(m["bf16_tflops"])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed regions run."""

    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self):
        self.rows, self.active, self._stop = [], False, False
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop:
            if self.active:
                try:
                    out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                         capture_output=True, text=True, timeout=5).stdout.strip()
                    if out:
                        self.rows.append([c.strip() for c in out.splitlines()[0].split(",")])
                except Exception:
                    pass
            time.sleep(0.1)

    def start(self):
        self.thread.start()

    def stop(self):
        self._stop = True

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no sample"]}
        sm = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows if len(r) > 2 + i)]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.rows)}


def model_folder(seed=0):
    """The random-weights model folder, made once per machine under the temporary directory."""
    from vitna_anchor_b200.engine.loading import write_random_model
    cfg = dict(SIZES, architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu")
    tag = hashlib.sha256(json.dumps([cfg, seed], sort_keys=True).encode()).hexdigest()[:12]
    d = os.path.join(tempfile.gettempdir(), f"vitna_bench_model_{os.getuid()}_{tag}")
    if not os.path.exists(os.path.join(d, "done")):
        t0 = time.time()
        write_random_model(d, cfg, seed)
        open(os.path.join(d, "done"), "w").close()
        print(f"[bench] wrote random SmolLM2-{MODEL_NAME} weights to {d} in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return d


def random_prompts(n, length, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [[int(t) for t in rng.integers(0, SIZES["vocab_size"], length)] for _ in range(n)]


def decode_run(model_dir, batch, steps, warmup, clocks, with_e2e):
    """Tokens a second of decode steps at `batch`, each request from its own PROMPT_LEN-token prompt."""
    import torch
    from vitna_anchor_b200 import ops
    from vitna_anchor_b200.engine.engine import Engine
    from vitna_anchor_b200.engine.runner import StepEntry
    eng = Engine(model_dir, dtype="bfloat16", ctx=CONTEXT, parallel=batch, kv_block=KV_BLOCK, max_batch_tokens=PREFILL_TOKENS)
    room = CONTEXT - PROMPT_LEN - 2
    assert 2 * (steps + warmup) <= room, "steps + warmup do not fit the context"
    reqs = [eng.add_request(p, max_new=room) for p in random_prompts(batch, PROMPT_LEN, 1)]
    while any(r.remaining > 1 or not r.output for r in reqs):     # prompts, untimed
        eng.step()
    out = {}
    if with_e2e:
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks.active = True
        t0 = time.perf_counter()
        ev0.record()
        for _ in range(steps):
            eng.step()                      # host ids in (pinned staging -> device), sampled ids out (device -> host)
        ev1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        clocks.active = False
        n_groups = len(eng.runner.cache.groups)
        meta_ints = 7 * batch + 1 + n_groups * (batch + batch * eng.runner.max_blocks)
        eng.flush()                         # the last step's ids (the engine runs a step ahead of the host's copy of them)
        out["e2e"] = {"value": batch * steps / wall, "unit": "tokens/s", "h2d_bytes_per_step": meta_ints * 4,
                      "d2h_bytes_per_step": batch * 4, "ms_per_step": wall / steps * 1e3,
                      "device_ms_per_step": ev0.elapsed_time(ev1) / steps}
    # the step function alone: fixed tokens, nothing read back
    runner = eng.runner
    entries = [StepEntry(r.request_id, [r.tokens[-1]], [0]) for r in reqs]
    ids = torch.empty(batch, dtype=torch.int32, device="cuda")
    for _ in range(warmup):
        ops.argmax_rows(runner.step(entries), ids)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ops.launch_count()
    clocks.active = True
    if PROFILE_REGION == "decode":
        torch.cuda.profiler.start()
    ev0.record()
    for _ in range(steps):
        ops.argmax_rows(runner.step(entries), ids)
    ev1.record()
    torch.cuda.synchronize()
    if PROFILE_REGION == "decode":
        torch.cuda.profiler.stop()
    clocks.active = False
    ms = ev0.elapsed_time(ev1) / steps
    ctx_mean = sum(runner.length(r.request_id) for r in reqs) / batch - steps / 2.0
    kv_bytes = runner.cache.bytes_per_token() * ctx_mean * batch
    out.update(ms_per_step=ms, value=batch * 1e3 / ms, launches=ops.launch_count() - launches0,
               bytes=eng.model.step_weight_bytes() + kv_bytes, context_mean=ctx_mean)
    del eng
    torch.cuda.empty_cache()
    return out


def prefill_run(model_dir, clocks, repeats=5):
    import torch
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    model = load_model(model_dir, "bfloat16")
    runner = ModelRunner(model, page_size=KV_BLOCK, num_pages=2 * PREFILL_TOKENS // KV_BLOCK, max_requests=2,
                         max_batch_tokens=PREFILL_TOKENS, max_model_len=CONTEXT)
    prompt = random_prompts(1, PREFILL_TOKENS, 2)[0]
    times, host = [], []
    for i in range(repeats + 3):
        runner.open(i)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks.active = i >= 3
        if PROFILE_REGION == "prefill" and i == repeats + 2:
            torch.cuda.profiler.start()
        t0 = time.perf_counter()
        ev0.record()
        runner.step([StepEntry(i, prompt, [PREFILL_TOKENS - 1])])
        ev1.record()
        host_ms = (time.perf_counter() - t0) * 1e3          # time to issue the step's launches
        torch.cuda.synchronize()
        if PROFILE_REGION == "prefill" and i == repeats + 2:
            torch.cuda.profiler.stop()
        clocks.active = False
        if i >= 3:
            times.append(ev0.elapsed_time(ev1))
            host.append(host_ms)
        runner.close(i)
    ms = sorted(times)[len(times) // 2]
    c = SIZES
    T, L, H, I = PREFILL_TOKENS, c["num_hidden_layers"], c["hidden_size"], c["intermediate_size"]
    qd, kvd = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    per_layer = H * (qd + 2 * kvd) + qd * H + 3 * H * I
    flops = 2.0 * T * per_layer * L + L * 4.0 * qd * T * (T + 1) / 2.0 + 2.0 * H * c["vocab_size"]
    return {"value": T * 1e3 / ms, "tokens": T, "ms": ms, "flops": flops, "host_issue_ms": sorted(host)[len(host) // 2]}


def gemm_run(pk, M=2048, reps=20):
    """TFLOP/s of the tcgen05 product at the projection shapes of SmolLM2-135M / 360M / 1.7B, M rows of activations.
    Operands are rotated through a set larger than L2 so that no launch finds its weights cached."""
    import torch
    from vitna_anchor_b200 import ops
    shapes = {"135M qkv": (960, 576), "135M gate_up": (3072, 576), "135M down": (576, 1536),
              "360M gate_up": (5120, 960), "360M down": (960, 2560),
              "1.7B qkv": (6144, 2048), "1.7B o": (2048, 2048), "1.7B gate_up": (16384, 2048), "1.7B down": (2048, 8192)}
    out = {}
    for name, (N, K) in shapes.items():
        copies = max(2, int(160e6 // (N * K * 2)) + 1)
        ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        for i in range(3):
            ops.linear_tcgen05(x, ws[i % copies], y, ops.LINEAR_SAME)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(reps):
            ops.linear_tcgen05(x, ws[i % copies], y, ops.LINEAR_SAME)
        ev1.record()
        torch.cuda.synchronize()
        ops.check_device_errors()
        us = ev0.elapsed_time(ev1) * 1e3 / reps
        tf = 2.0 * M * N * K / (us * 1e-6) / 1e12
        out[name] = {"us": round(us, 1), "tflops": round(tf, 1), "frac": round(tf / pk["bf16_tflops"], 3)}
        del ws
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="135M", choices=sorted(MODELS), help="layer sizes: SmolLM2-135M (the default), 360M or 1.7B")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64 and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="run the prefill measurement alone (for profiling)")
    ap.add_argument("--profile-region", default="", choices=["", "decode", "prefill"],
                    help="bracket the timed decode steps (or the last prefill) with cudaProfilerStart/Stop, for ncu --profile-from-start off")
    ap.add_argument("--only-gemm", action="store_true", help="time the tcgen05 product alone at the models' shapes, M = 2,048")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "pip cannot install the reference offline: it is a C program with a "
                          "Node wrapper and has neither setup.py nor pyproject.toml"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {a.gpus} is not supported by this engine")
        return 2
    a.warmup = max(a.warmup, 3)
    global MODEL_NAME, PROFILE_REGION
    MODEL_NAME = a.model
    PROFILE_REGION = a.profile_region
    SIZES.clear()
    SIZES.update(MODELS[a.model])
    import torch
    from vitna_anchor_b200 import ops
    ops.lib()
    pk = peaks()
    model_dir = model_folder()
    clocks = ClockSampler()
    clocks.start()
    if a.only_gemm:
        print(json.dumps({"gemm_m2048": gemm_run(pk)}))
        return 0
    if a.only_prefill:
        pf = prefill_run(model_dir, clocks, repeats=3)
        clocks.stop()
        print(json.dumps({"prefill": {"value": pf["value"], "tokens": pf["tokens"], "ms": pf["ms"], "host_issue_ms": pf["host_issue_ms"],
                                      "frac": pf["flops"] / (pf["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12)}}))
        return 0
    main_run = decode_run(model_dir, a.batch, a.steps, a.warmup, clocks, with_e2e=True)
    points, prefill = {}, None
    if not a.no_points:
        k = min(a.steps, 64)
        points["decode_b1"] = decode_run(model_dir, 1, k, a.warmup, clocks, False)["value"]
        points["decode_b64"] = decode_run(model_dir, 64, k, a.warmup, clocks, False)["value"]
        prefill = prefill_run(model_dir, clocks)
    clocks.stop()
    achieved = main_run["bytes"] / (main_run["ms_per_step"] * 1e-3) / 1e9
    line = {
        "metric": f"decode tokens/s, SmolLM2-{MODEL_NAME} random weights, batch {a.batch} from 2,048-token prompts", "value": main_run["value"],
        "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": main_run["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and uniform-random token ids", "impl": "ours",
        "config": {"model": f"SmolLM2-{MODEL_NAME}", "layers": SIZES["num_hidden_layers"], "layers_of_model": SIZES["num_hidden_layers"],
                   "hidden": SIZES["hidden_size"],
                   "heads": SIZES["num_attention_heads"], "kv_heads": SIZES["num_key_value_heads"], "head_dim": SIZES["head_dim"],
                   "intermediate": SIZES["intermediate_size"], "vocab": SIZES["vocab_size"], "global_batch": a.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "context_mean": round(main_run["context_mean"]),
                   "kv_block": KV_BLOCK, "parallelism": "1 GPU", "l2": "inputs larger than L2", "peaks": pk["source"]},
        "e2e": main_run.get("e2e"), "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
        "points": points, "clocks": clocks.summary(),
    }
    if prefill:
        line["prefill"] = {"value": prefill["value"], "tokens": prefill["tokens"], "ms": prefill["ms"],
                           "frac": prefill["flops"] / (prefill["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12)}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
