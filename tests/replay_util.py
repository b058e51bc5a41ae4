"""Driving bin/trace_run from tests: schedules of steps, and the logits it wrote."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Replay:
    """One trace_run process.  run(steps) feeds steps one by one, waiting for `done <step>` after each,
    and returns {(request id, position): logits row}."""

    def __init__(self, model_dir, dtype, out_dir, max_tokens, kv_block=None, max_requests=None, plugins=None):
        self.out_dir = str(out_dir)
        cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", self.out_dir, "--max-tokens", str(max_tokens)]
        if kv_block is not None:
            cmd += ["--kv-block", str(kv_block)]
        if max_requests is not None:
            cmd += ["--max-requests", str(max_requests)]
        env = dict(os.environ)
        if plugins:          # architectures defined under tests/: the child imports them by name
            env["VITNA_ANCHOR_PLUGINS"] = plugins
            env["PYTHONPATH"] = os.path.dirname(os.path.abspath(__file__)) + os.pathsep + env.get("PYTHONPATH", "")
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        self.next_step = 0
        self.position = {}

    def run(self, steps, vocab):
        """steps: list of (entries, end) with entries = [(id, tokens, want)]."""
        got = {}
        for entries, end in steps:
            n = self.next_step
            self.next_step += 1
            rec = {"step": n, "entries": [{"id": i, "tokens": list(map(int, t)), "want": list(map(int, w))} for i, t, w in entries],
                   "end": list(end)}
            self.proc.stdin.write(json.dumps(rec) + "\n")
            self.proc.stdin.flush()
            line = self.proc.stdout.readline()
            assert line.strip() == f"done {n}", f"trace_run said {line!r} (exit {self.proc.poll()})"
            wanted = sum(len(w) for _, _, w in entries)
            path = os.path.join(self.out_dir, f"{n}.f32")
            if wanted:
                rows = np.fromfile(path, "<f4").reshape(wanted, vocab)
                r = 0
                for i, t, w in entries:
                    base = self.position.get(i, 0)
                    for place in w:
                        got[(i, base + place)] = rows[r]
                        r += 1
            else:
                assert not os.path.exists(path)
            for i, t, _ in entries:
                self.position[i] = self.position.get(i, 0) + len(t)
            for i in end:
                self.position.pop(i, None)
        return got

    def close(self):
        self.proc.stdin.close()
        code = self.proc.wait(timeout=120)
        assert code == 0, f"trace_run exited with {code}"


def whole(rid, ids):
    return [([(rid, ids, range(len(ids)))], [rid])]


def tail_one_by_one(rid, ids, tail=32):
    head = max(1, len(ids) - tail)
    steps = [([(rid, ids[:head], range(head))], [])]
    for p in range(head, len(ids)):
        steps.append(([(rid, ids[p:p + 1], [0])], []))
    steps[-1] = (steps[-1][0], [rid])
    return steps


def changing_portions(rid, ids, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 64, 11)):
    steps, p, k = [], 0, 0
    while p < len(ids):
        n = min(sizes[k % len(sizes)], len(ids) - p)
        if len(ids) - p - n == 1:       # never leave a single token: the smallest portion is two
            n += 1
        steps.append(([(rid, ids[p:p + n], range(n))], []))
        p += n
        k += 1
    steps[-1] = (steps[-1][0], [rid])
    return steps


def mixed(requests, prompt_part, rng, live_max=4, portions=(2, 12), one_prompt_at_a_time=False):
    """requests: {id: ids}; the first prompt_part[id] tokens go in portions of portions[0]..portions[1]-1 tokens
    (2..11 unless given), the rest one by one.  Up to live_max requests are live; a live request is sometimes
    left out of a step.  one_prompt_at_a_time: a request is let in only when every live one is past its prompt
    part, so that its portions run beside the decoded tokens of the others."""
    waiting = list(requests)
    live, pos, steps = [], {}, []
    while waiting or live:
        while (waiting and len(live) < live_max
               and not (one_prompt_at_a_time and any(pos[r] < prompt_part[r] for r in live))):
            rid = waiting.pop(0)
            live.append(rid)
            pos[rid] = 0
        entries, end = [], []
        for rid in list(live):
            ids = requests[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue
            p = pos[rid]
            if p < prompt_part[rid]:
                n = min(int(rng.integers(portions[0], portions[1])), prompt_part[rid] - p)
                if prompt_part[rid] - p - n == 1:
                    n += 1
            else:
                n = 1
            n = min(n, len(ids) - p)
            entries.append((rid, ids[p:p + n], range(n)))
            pos[rid] = p + n
            if pos[rid] == len(ids):
                end.append(rid)
                live.remove(rid)
        if entries:
            steps.append((entries, end))
    return steps
