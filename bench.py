#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]
                    [--model 135M|360M|1.7B] [--workload decode|mixed|prefill8k]

The default run is SmolLM2-135M's sizes with random weights (N(0, 0.02), norm weights 1, seed 0) in
bfloat16, a batch of 8 requests each decoding from its own 2,048-token random prompt, cache context
4,096, pages of 16.  A "step" is one decode step of the whole batch.

  value     decoded tokens a second through the step function (CUDA events around K steps)
  e2e       the same through the Python entry point (Engine.step: host token ids in, host token ids out)
  prefill   one 2,048-token prompt in one step: tokens a second, and flops / time / peak
  roofline  bytes the decode step must read (every weight once, the live requests' cache) / its time / peak
  points    decoded tokens a second at batch 1 and 64 (and batch 1 end to end, the reference arm's case); the
            1.7B sizes' batch-64 decode and prefills of 2,048 and 8,192 tokens; the 360M sizes' mixed workload
  roofline_points   the fraction of the peak for each of those

--workload mixed: 32 requests with prompts of 16..2,048 random tokens (seeded), prompts run in portions of at
most 512 tokens beside the decoded tokens of the others, 128 new tokens each, through Engine.step.
--workload prefill8k: one 8,192-token prompt, in one step and in portions of 2,048 through the scheduler.

--impl reference builds nothing of this repository's engine: it runs the unmodified reference program
(baseline/_ref/engine/vitna-anchor, built from the reference's own Makefile with VITNA_CUDA=1) through its stock
command line, `generate --ids-file F --max-new N --greedy --timing --device cuda --ctx 4096`, on the same seeded
SmolLM2-135M folder, and reads its own timing line, as the reference's scripts/bench-decode.mjs does.  That command
line has one request at a time, so its figures are batch 1, in float32 (the reference's kernels compute in float32).

Every step reads more than the 126 MB of L2 (weights 269 MB alone), so no flush is needed between
timed iterations.  Peaks come from MEASURED_PEAKS.json when the driver wrote it, else the fallback
(6.65 TB/s, 1.59 PFLOP/s bf16).
"""
import argparse
import hashlib
import json
import os
import re
import shutil
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


def config_json(sizes):
    return dict(sizes, architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu")


def model_folder(seed=0):
    """The random-weights model folder, made once per machine under the temporary directory."""
    from vitna_anchor_b200.engine.loading import write_random_model
    cfg = config_json(SIZES)
    tag = hashlib.sha256(json.dumps([cfg, seed], sort_keys=True).encode()).hexdigest()[:12]
    d = os.path.join(tempfile.gettempdir(), f"vitna_bench_model_{os.getuid()}_{tag}")
    if not os.path.exists(os.path.join(d, "done")):
        t0 = time.time()
        write_random_model(d, cfg, seed)
        open(os.path.join(d, "done"), "w").close()
        print(f"[bench] wrote random SmolLM2-{MODEL_NAME} weights to {d} in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return d


def random_prompts(n, length, seed, vocab=None):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [[int(t) for t in rng.integers(0, vocab or SIZES["vocab_size"], length)] for _ in range(n)]


def decode_run(model, batch, steps, warmup, clocks, with_e2e):
    """Tokens a second of decode steps at `batch`, each request from its own PROMPT_LEN-token prompt.
    model: a model folder, or a model already on the device."""
    import torch
    from vitna_anchor_b200 import ops
    from vitna_anchor_b200.engine.engine import Engine
    from vitna_anchor_b200.engine.runner import StepEntry
    eng = Engine(model, dtype="bfloat16", ctx=CONTEXT, parallel=batch, kv_block=KV_BLOCK, max_batch_tokens=PREFILL_TOKENS)
    room = CONTEXT - PROMPT_LEN - 2
    assert 2 * (steps + warmup) <= room, "steps + warmup do not fit the context"
    reqs = [eng.add_request(p, max_new=room) for p in random_prompts(batch, PROMPT_LEN, 1, eng.model.vocab_size)]
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
    runner.check(sync=False)
    ms = ev0.elapsed_time(ev1) / steps
    ctx_mean = sum(runner.length(r.request_id) for r in reqs) / batch - steps / 2.0
    kv_bytes = runner.cache.bytes_per_token() * ctx_mean * batch
    nbytes = eng.model.step_weight_bytes() + kv_bytes
    out.update(ms_per_step=ms, value=batch * 1e3 / ms, launches=ops.launch_count() - launches0,
               bytes=nbytes, context_mean=ctx_mean, gbs=nbytes / (ms * 1e-3) / 1e9)
    del eng, runner
    torch.cuda.empty_cache()
    return out


def prefill_flops(sizes, T):
    c = sizes
    L, H, I = c["num_hidden_layers"], c["hidden_size"], c["intermediate_size"]
    qd, kvd = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    per_layer = H * (qd + 2 * kvd) + qd * H + 3 * H * I
    return 2.0 * T * per_layer * L + L * 4.0 * qd * T * (T + 1) / 2.0 + 2.0 * H * c["vocab_size"]


def prefill_run(model, sizes, clocks, tokens=PREFILL_TOKENS, portion=0, repeats=5):
    """One prompt of `tokens` tokens: in one step (portion 0), or in portions of `portion` tokens, one step each."""
    import torch
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    if isinstance(model, str):
        model = load_model(model, "bfloat16")
    per_step = portion or tokens
    runner = ModelRunner(model, page_size=KV_BLOCK, num_pages=2 * tokens // KV_BLOCK, max_requests=2,
                         max_batch_tokens=per_step, max_model_len=max(CONTEXT, tokens))
    prompt = random_prompts(1, tokens, 2, model.vocab_size)[0]
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
        for p in range(0, tokens, per_step):
            n = min(per_step, tokens - p)
            runner.step([StepEntry(i, prompt[p:p + n], [n - 1] if p + n == tokens else [])])
        ev1.record()
        host_ms = (time.perf_counter() - t0) * 1e3          # time to issue the step's launches
        torch.cuda.synchronize()
        if PROFILE_REGION == "prefill" and i == repeats + 2:
            torch.cuda.profiler.stop()
        clocks.active = False
        runner.check(sync=False)
        if i >= 3:
            times.append(ev0.elapsed_time(ev1))
            host.append(host_ms)
        runner.close(i)
    ms = sorted(times)[len(times) // 2]
    del runner
    torch.cuda.empty_cache()
    return {"value": tokens * 1e3 / ms, "tokens": tokens, "ms": ms, "flops": prefill_flops(sizes, tokens),
            "host_issue_ms": sorted(host)[len(host) // 2]}


def mixed_run(model, clocks, requests=32, new_tokens=128, portion=512, seed=4):
    """BASELINE configs[3]'s workload: `requests` requests with prompts of 16..2,048 random tokens, prompts run in
    portions of at most `portion` tokens beside the decoded tokens of the others, `new_tokens` new tokens each;
    everything through Engine.step (host ids in, host ids out)."""
    import numpy as np
    import torch
    from vitna_anchor_b200 import ops
    from vitna_anchor_b200.engine.engine import Engine
    eng = Engine(model, dtype="bfloat16", ctx=CONTEXT, parallel=requests, kv_block=KV_BLOCK, max_batch_tokens=portion + 64,
                 max_prompt_portion=portion)
    rng = np.random.default_rng(seed)
    lengths = [int(n) for n in rng.integers(16, 2049, requests)]

    def once():
        prompts = [[int(t) for t in rng.integers(0, eng.model.vocab_size, n)] for n in lengths]
        reqs = [eng.add_request(p, max_new=new_tokens) for p in prompts]
        torch.cuda.synchronize()
        launches0, steps0 = ops.launch_count(), eng.runner.steps_run
        t0 = time.perf_counter()
        while eng.scheduler.has_work():
            eng.step()
        eng.flush()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        assert all(len(r.output) == new_tokens for r in reqs)
        return wall, eng.runner.steps_run - steps0, ops.launch_count() - launches0
    # warm-up: the same lengths, so the same shapes of steps come again; a shape is captured into a graph at its second
    # coming, so two rounds go before the timed one
    rounds = [once()[0], once()[0]]
    clocks.active = True
    wall, steps, launches = once()
    clocks.active = False
    out = {"value": requests * new_tokens / wall, "unit": "new tokens/s", "all_tokens_per_s": (sum(lengths) + requests * new_tokens) / wall,
           "seconds": wall, "steps": steps, "launches": launches, "prompt_tokens": sum(lengths), "requests": requests,
           "new_tokens_each": new_tokens, "portion": portion, "graph_replays": eng.runner.graph_replays,
           "warmup_round_seconds": rounds, "graphs": len(eng.runner._mixed_graphs) + len(eng.runner._decode_graphs)}
    del eng
    torch.cuda.empty_cache()
    return out


def gemm_run(pk, M=2048, reps=20):
    """TFLOP/s of the tcgen05 product at the projection shapes of SmolLM2-135M / 360M / 1.7B, M rows of activations, with the
    epilogue the model uses there: gate_up with SwiGLU, o and down adding into the float32 residual stream, qkv plain.
    Operands are rotated through a set larger than L2 so that no launch finds its weights cached."""
    import torch
    from vitna_anchor_b200 import ops
    shapes = {"135M qkv": (960, 576, "same"), "135M o": (576, 576, "acc"), "135M gate_up": (3072, 576, "swiglu"), "135M down": (576, 1536, "acc"),
              "360M qkv": (1600, 960, "same"), "360M gate_up": (5120, 960, "swiglu"), "360M down": (960, 2560, "acc"),
              "1.7B qkv": (6144, 2048, "same"), "1.7B o": (2048, 2048, "acc"), "1.7B gate_up": (16384, 2048, "swiglu"),
              "1.7B down": (2048, 8192, "acc")}
    out = {}
    for name, (N, K, kind) in shapes.items():
        copies = max(2, int(160e6 // (N * K * 2)) + 1)
        ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        if kind == "swiglu":
            y = torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda")
            run = lambda w: ops.linear_tcgen05_swiglu(x, w, y)
        elif kind == "acc":
            y = torch.zeros(M, N, dtype=torch.float32, device="cuda")
            run = lambda w: ops.linear_tcgen05(x, w, y, ops.LINEAR_ACC_F32)
        else:
            y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            run = lambda w: ops.linear_tcgen05(x, w, y, ops.LINEAR_SAME)
        for i in range(3):
            run(ws[i % copies])
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()          # the launches are replayed from a graph, as in a step: the host's pace does not count
        with torch.cuda.graph(graph):
            for i in range(reps):
                run(ws[i % copies])
        graph.replay()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        graph.replay()
        ev1.record()
        torch.cuda.synchronize()
        ops.check_device_errors()
        us = ev0.elapsed_time(ev1) * 1e3 / reps
        tf = 2.0 * M * N * K / (us * 1e-6) / 1e12
        out[name] = {"us": round(us, 1), "tflops": round(tf, 1), "frac": round(tf / pk["bf16_tflops"], 3)}
        del ws
    return out


# ---------------------------------------------------------------------------------------------------------------
# The reference arm
# ---------------------------------------------------------------------------------------------------------------

REF_DIR = os.path.join(ROOT, "baseline", "_ref", "engine")
REF_EXE = os.path.join(REF_DIR, "vitna-anchor")


def reference_source():
    """Where the reference's engine sources lie: VITNA_REFERENCE_SOURCE, else the `reference_path` that BASELINE.json names."""
    env = os.environ.get("VITNA_REFERENCE_SOURCE")
    if env:
        return env
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as fh:
            return os.path.join(json.load(fh)["reference_path"], "engine")
    except (OSError, KeyError, ValueError):
        return ""


REF_SOURCE = reference_source()


def byte_level_tokenizer_json():
    """The smallest tokenizer.json the reference's `generate` accepts (it loads one even for --ids-file): a
    byte-level BPE with the 256 byte tokens and no merges.  It is a data file beside config.json; the prompt is given
    as ids and the ids that come out are never turned into text by this bench."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b); cs.append(256 + n); n += 1
    vocab = {chr(c): i for i, (_, c) in enumerate(sorted(zip(bs, cs)))}
    return {"version": "1.0", "added_tokens": [], "normalizer": None,
            "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": True},
            "post_processor": None, "decoder": {"type": "ByteLevel"},
            "model": {"type": "BPE", "dropout": None, "unk_token": None, "vocab": vocab, "merges": []}}


def build_reference():
    """The reference program for CUDA, built by its own Makefile from a copy of its sources (the source tree is
    read-only and the Makefile writes objects beside it).  Returns None, or why it cannot be had."""
    if os.path.exists(REF_EXE):
        return None
    if not os.path.isdir(REF_SOURCE):
        return f"{REF_EXE} is not built and the reference's sources are not on this machine"
    if not shutil.which("nvcc") and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        return "nvcc is not on this machine, so the reference's CUDA path cannot be built"
    os.makedirs(os.path.dirname(REF_DIR), exist_ok=True)
    if not os.path.isdir(REF_DIR):
        shutil.copytree(REF_SOURCE, REF_DIR)
    env = dict(os.environ, PATH=os.environ.get("PATH", "") + os.pathsep + "/usr/local/cuda/bin")
    p = subprocess.run(["make", "VITNA_CUDA=1", "CUDA_ARCH=sm_100", "CC=gcc", "-j8"], cwd=REF_DIR, env=env, capture_output=True, text=True)
    if p.returncode != 0 or not os.path.exists(REF_EXE):
        return "the reference's Makefile failed: " + (p.stderr.strip().splitlines() or ["no message"])[-1][:200]
    return None


def reference_run(steps, warmup):
    why = build_reference()
    if why:
        return {"impl": "reference", "unavailable": why}
    model_dir = model_folder()
    tok = os.path.join(model_dir, "tokenizer.json")
    if not os.path.exists(tok):
        with open(tok, "w") as f:
            json.dump(byte_level_tokenizer_json(), f)
    ids_file = os.path.join(model_dir, "bench_prompt_ids.txt")
    with open(ids_file, "w") as f:
        f.write(",".join(str(t) for t in random_prompts(1, PROMPT_LEN, 1)[0]))
    new = max(steps, 16) + 1
    cmd = [REF_EXE, "generate", "--model", model_dir, "--ids-file", ids_file, "--max-new", str(new), "--greedy", "--timing",
           "--device", "cuda", "--ctx", str(CONTEXT)]
    pat = re.compile(r"timing: (\d+) prompt tokens in ([\d.]+) ms; (\d+) tokens after the first new one in ([\d.]+) ms, ([\d.]+) ms each")
    runs, prompts, walls = [], [], []
    clocks = ClockSampler()
    clocks.start()
    for i in range(1 + 3):                   # one run thrown away, then the median of three (the reference's method)
        clocks.active = i > 0
        t0 = time.perf_counter()
        try:
            p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        except subprocess.TimeoutExpired:
            clocks.stop()
            return {"impl": "reference", "unavailable": "the reference's generate command did not end within 600 s on this GPU"}
        clocks.active = False
        m = pat.search(p.stderr)
        if p.returncode != 0 or not m:
            clocks.stop()
            tail = (p.stderr.strip().splitlines() or ["no message"])[-1][:200]
            return {"impl": "reference", "unavailable": f"the reference's generate command exited {p.returncode}: {tail}"}
        if i > 0:
            runs.append(float(m.group(5))); prompts.append(float(m.group(2))); walls.append(time.perf_counter() - t0)
    clocks.stop()
    ms = sorted(runs)[len(runs) // 2]
    pms = sorted(prompts)[len(prompts) // 2]
    c = SIZES
    return {
        "metric": "decode tokens/s, SmolLM2-135M random weights, batch 1 from a 2,048-token prompt (the reference's own command line)",
        "value": 1e3 / ms, "unit": "tokens/s", "n_gpus": 1, "steps": new - 1, "warmup": 1, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32 arithmetic on bf16 weights (the reference's CUDA path)",
        "data": "synthetic: the same seeded random weights and prompt as this repository's arm", "impl": "reference",
        "config": {"model": "SmolLM2-135M", "layers": c["num_hidden_layers"], "layers_of_model": c["num_hidden_layers"], "hidden": c["hidden_size"],
                   "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
                   "intermediate": c["intermediate_size"], "vocab": c["vocab_size"], "global_batch": 1, "seq_len": CONTEXT,
                   "prompt_len": PROMPT_LEN, "parallelism": "1 GPU", "same_config": False,
                   "differs": "batch 1 (ours: 8) and float32 arithmetic; compare with points.e2e_b1 and prefill of our arm"},
        # its timing is taken on the host around whole steps (logits to the host, the choice there): it is end to end
        "e2e": {"value": 1e3 / ms, "unit": "tokens/s", "ms_per_step": ms, "h2d_bytes_per_step": 12, "d2h_bytes_per_step": c["vocab_size"] * 4},
        "prefill": {"value": PROMPT_LEN * 1e3 / pms, "tokens": PROMPT_LEN, "ms": pms},
        "gpu_launches": None, "command": " ".join(cmd), "run_seconds": walls, "clocks": clocks.summary(),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="135M", choices=sorted(MODELS), help="layer sizes: SmolLM2-135M (the default), 360M or 1.7B")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed", "prefill8k"],
                    help="decode (the default line), mixed (32 requests, 512-token portions beside decodes), prefill8k")
    ap.add_argument("--no-points", action="store_true", help="skip the other batches, models and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="run the prefill measurement alone (for profiling)")
    ap.add_argument("--profile-region", default="", choices=["", "decode", "prefill"],
                    help="bracket the timed decode steps (or the last prefill) with cudaProfilerStart/Stop, for ncu --profile-from-start off")
    ap.add_argument("--only-gemm", action="store_true", help="time the tcgen05 product alone at the models' shapes, M = 2,048")
    a = ap.parse_args()
    if a.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {a.gpus} is not supported by this engine")
        return 2
    a.warmup = max(a.warmup, 3)
    global MODEL_NAME, PROFILE_REGION
    if a.impl == "reference":
        print(json.dumps(reference_run(a.steps, a.warmup)))
        return 0
    MODEL_NAME = a.model
    PROFILE_REGION = a.profile_region
    SIZES.clear()
    SIZES.update(MODELS[a.model])
    import torch
    from vitna_anchor_b200 import ops
    from vitna_anchor_b200.engine.loading import random_model_on_device
    ops.lib()
    pk = peaks()
    clocks = ClockSampler()
    clocks.start()
    if a.only_gemm:
        print(json.dumps({"gemm_m2048": gemm_run(pk)}))
        return 0
    if a.workload == "mixed":
        model = random_model_on_device(config_json(SIZES), 0) if a.model != "135M" else model_folder()
        r = mixed_run(model, clocks)
        clocks.stop()
        print(json.dumps({"metric": f"new tokens/s, SmolLM2-{a.model} random weights, 32 requests with prompts of 16..2,048 tokens in portions "
                          "of 512 beside decodes, 128 new tokens each, through Engine.step", "impl": "ours", "dtype": "bf16", **r,
                          "clocks": clocks.summary()}))
        return 0
    if a.workload == "prefill8k":
        model = random_model_on_device(config_json(SIZES), 0)
        one = prefill_run(model, SIZES, clocks, tokens=8192, repeats=3)
        cut = prefill_run(model, SIZES, clocks, tokens=8192, portion=2048, repeats=3)
        clocks.stop()
        f = lambda r: {"value": r["value"], "ms": r["ms"], "frac": r["flops"] / (r["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12)}
        print(json.dumps({"metric": f"prefill tokens/s of one 8,192-token prompt, SmolLM2-{a.model} random weights", "impl": "ours",
                          "one_step": f(one), "portions_of_2048": f(cut), "clocks": clocks.summary()}))
        return 0
    if a.only_prefill:
        pf = prefill_run(model_folder(), SIZES, clocks, repeats=3)
        clocks.stop()
        print(json.dumps({"prefill": {"value": pf["value"], "tokens": pf["tokens"], "ms": pf["ms"], "host_issue_ms": pf["host_issue_ms"],
                                      "frac": pf["flops"] / (pf["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12)}}))
        return 0
    model_dir = model_folder()
    main_run = decode_run(model_dir, a.batch, a.steps, a.warmup, clocks, with_e2e=True)
    points, fracs, prefill = {}, {}, None
    if not a.no_points:
        k = min(a.steps, 64)
        b1 = decode_run(model_dir, 1, k, a.warmup, clocks, True)
        b64 = decode_run(model_dir, 64, k, a.warmup, clocks, False)
        points.update(decode_b1=b1["value"], decode_b64=b64["value"], e2e_b1=b1["e2e"]["value"])
        fracs.update(decode_b1=b1["gbs"] / pk["hbm_gbs"], decode_b64=b64["gbs"] / pk["hbm_gbs"])
        prefill = prefill_run(model_dir, SIZES, clocks)
        if a.model == "135M":
            # the larger models of BASELINE.json, with weights drawn on the device (no checkpoint is written)
            big = random_model_on_device(config_json(MODELS["1.7B"]), 0)
            d = decode_run(big, 64, min(k, 32), a.warmup, clocks, False)
            p2 = prefill_run(big, MODELS["1.7B"], clocks, repeats=3)
            p8 = prefill_run(big, MODELS["1.7B"], clocks, tokens=8192, portion=2048, repeats=3)
            points.update({"1p7b_decode_b64": d["value"], "1p7b_prefill_2048": p2["value"], "1p7b_prefill_8192": p8["value"]})
            fracs.update({"1p7b_decode_b64": d["gbs"] / pk["hbm_gbs"],
                          "1p7b_prefill_2048": p2["flops"] / (p2["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12),
                          "1p7b_prefill_8192": p8["flops"] / (p8["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12)})
            del big
            torch.cuda.empty_cache()
            mid = random_model_on_device(config_json(MODELS["360M"]), 0)
            mx = mixed_run(mid, clocks)
            points["360m_mixed_new_tokens_per_s"] = mx["value"]
            points["360m_mixed_all_tokens_per_s"] = mx["all_tokens_per_s"]
            del mid
            torch.cuda.empty_cache()
    clocks.stop()
    achieved = main_run["gbs"]
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
        "points": points, "roofline_points": fracs, "clocks": clocks.summary(),
    }
    if prefill:
        line["prefill"] = {"value": prefill["value"], "tokens": prefill["tokens"], "ms": prefill["ms"],
                           "frac": prefill["flops"] / (prefill["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12)}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
