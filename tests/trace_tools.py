"""Drives ``bin/trace_run`` as a child process and builds traces for the ways of cutting work."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# (step, row in the step's file) -> (request id, position)
Where = List[Tuple[int, int, str, int]]


class TraceRunner:
    def __init__(self, model_dir: str, dtype: str, out_dir: str, max_tokens: int, page_size: int,
                 max_requests: int = 8):
        self.out_dir = out_dir
        self.proc = subprocess.Popen(
            [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
             "--max-tokens", str(max_tokens), "--page-size", str(page_size), "--max-requests", str(max_requests)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)

    def run(self, steps: Sequence[dict]) -> None:
        for step in steps:
            self.proc.stdin.write(json.dumps(step) + "\n")
            self.proc.stdin.flush()
            line = self.proc.stdout.readline()
            if line.strip() != f"done {step['step']}":
                rest = self.proc.stdout.read()
                raise AssertionError(f"trace_run answered {line!r}{rest!r} to step {step['step']} "
                                     f"(exit {self.proc.poll()})")

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)

    def logits(self, step: int, vocab: int) -> np.ndarray:
        return np.fromfile(os.path.join(self.out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab)


class TraceBuilder:
    """Collects steps and remembers which (request, position) every wanted row is."""

    def __init__(self, first_step: int = 0):
        self.steps: List[dict] = []
        self.where: Where = []
        self._next = first_step
        self._fed: Dict[str, int] = {}

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], end: Sequence[str] = ()) -> int:
        """entries: (request id, tokens, wanted places)."""
        number = self._next
        self._next += 1
        row = 0
        out = []
        for rid, tokens, want in entries:
            start = self._fed.get(rid, 0)
            for w in want:
                self.where.append((number, row, rid, start + w))
                row += 1
            self._fed[rid] = start + len(tokens)
            out.append({"id": rid, "tokens": list(map(int, tokens)), "want": list(map(int, want))})
        for rid in end:
            self._fed.pop(rid, None)
        self.steps.append({"step": number, "entries": out, "end": list(end)})
        return number


def cut_whole(b: TraceBuilder, rid: str, tokens: Sequence[int]) -> None:
    b.step([(rid, tokens, range(len(tokens)))], end=[rid])


def cut_decode_tail(b: TraceBuilder, rid: str, tokens: Sequence[int], tail: int = 32) -> None:
    head = len(tokens) - tail
    assert head >= 1
    b.step([(rid, tokens[:head], range(head))])
    for i in range(head, len(tokens)):
        b.step([(rid, tokens[i:i + 1], [0])], end=[rid] if i == len(tokens) - 1 else [])


def cut_portions(b: TraceBuilder, rid: str, tokens: Sequence[int], sizes: Sequence[int]) -> None:
    at, i = 0, 0
    while at < len(tokens):
        n = min(sizes[i % len(sizes)], len(tokens) - at)
        i += 1
        last = at + n == len(tokens)
        b.step([(rid, tokens[at:at + n], range(n))], end=[rid] if last else [])
        at += n


def cut_mixed(b: TraceBuilder, requests: Dict[str, Sequence[int]], sizes: Sequence[int], live: int = 4,
              seed: int = 0) -> None:
    """Up to ``live`` requests at a time.  A request is fed in portions until 12 tokens remain,
    then token by token, so portions of some run beside single tokens of others; a finished
    request is ended and the next one starts in the same step's slot."""
    rng = np.random.default_rng(seed)
    waiting = list(requests)
    running: Dict[str, int] = {}
    turn = 0
    while waiting or running:
        while waiting and len(running) < live:
            running[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(running):
            tokens, at = requests[rid], running[rid]
            left = len(tokens) - at
            if rng.random() < 0.2 and len(running) > 1:
                continue                       # left out of this step, goes on later
            n = 1 if left <= 12 else min(sizes[turn % len(sizes)], left - 12)
            turn += 1
            entries.append((rid, tokens[at:at + n], range(n)))
            running[rid] = at + n
            if at + n == len(tokens):
                end.append(rid)
                del running[rid]
        if entries:
            b.step(entries, end=end)
