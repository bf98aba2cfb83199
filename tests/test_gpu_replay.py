"""Trace replay through bin/trace_run, compared with the plain implementation: each request
alone and whole; with its last 32 tokens one by one; in batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots and pages are used
again.  float32 and bfloat16, both tiny configurations, plus a model whose attention is made
peaky so that a fault in masking or cache addressing cannot hide."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, TINY, close, prompts_for

pytestmark = pytest.mark.gpu

LENGTHS = [70, 33, 129, 45, 100, 64]      # crossing the 64-token page edge, longer than the windows of A and B
LENGTHS_C = [170, 33, 257, 45, 100, 64]   # for C: longer than its window of 96, several 64-row attention tiles


class Replay:
    """One trace_run process, driven step by step."""

    def __init__(self, model_dir, dtype, out_dir, max_tokens):
        self.out = str(out_dir)
        self.proc = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
             "--out", self.out, "--max-tokens", str(max_tokens)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.n = 0
        self.vocab = None

    def step(self, entries, end=()):
        sid = self.n
        self.n += 1
        rec = {"step": sid, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {sid}", f"trace_run answered {line!r} (exit code {self.proc.poll()})"
        wanted = sum(len(w) for _, _, w in entries)
        path = os.path.join(self.out, f"{sid}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
            return np.zeros((0, 0), dtype=np.float32)
        return np.fromfile(path, dtype="<f4").reshape(wanted, -1)

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


def run_all_cuttings(replay, requests, ref, dtype):
    """`ref[i]` = plain logits [len_i, V].  Returns the largest error seen."""
    worst = 0.0

    def check(got, want, what):
        nonlocal worst
        ok, err, tol = close(got, want, dtype)
        worst = max(worst, err)
        assert ok, f"{what}: error {err:.3g} > {tol:.3g}"

    # 1. each request alone and whole, every position wanted
    for i, toks in enumerate(requests):
        got = replay.step([(f"w{i}", toks, range(len(toks)))], end=[f"w{i}"])
        check(got, ref[i], f"request {i} whole")
    # 2. each request with its last 32 tokens one by one
    for i, toks in enumerate(requests):
        cut = max(1, len(toks) - 32)
        got = replay.step([(f"s{i}", toks[:cut], [cut - 1])])
        check(got, ref[i][cut - 1:cut], f"request {i} prefix")
        for p in range(cut, len(toks)):
            last = p == len(toks) - 1
            got = replay.step([(f"s{i}", [toks[p]], [0])], end=[f"s{i}"] if last else [])
            check(got, ref[i][p:p + 1], f"request {i} position {p} decoded alone")
        if cut == len(toks):
            replay.step([], end=[f"s{i}"])
    # 3. batches of unequal lengths: prompts of different sizes start together, then one token each;
    #    the shorter requests end earlier; the next batch reuses what they held
    for batch, prompt_lens in (([0, 1, 2], [40, 33, 65]), ([3, 4, 5, 1], [1, 64, 63, 7]), ([2, 0], [129, 5])):
        ids = {i: f"b{batch[0]}_{i}" for i in batch}
        entries = [(ids[i], requests[i][:n], [0, n - 1] if n > 1 else [0]) for i, n in zip(batch, prompt_lens)]
        ended = [ids[i] for i, n in zip(batch, prompt_lens) if n == len(requests[i])]
        got = replay.step(entries, end=ended)
        r = 0
        for i, n in zip(batch, prompt_lens):
            rows = [0, n - 1] if n > 1 else [0]
            check(got[r:r + len(rows)], ref[i][rows], f"batch {batch} prompt of request {i}")
            r += len(rows)
        pos = {i: n for i, n in zip(batch, prompt_lens) if n < len(requests[i])}
        while pos:
            live = sorted(pos)
            entries = [(ids[i], [requests[i][pos[i]]], [0]) for i in live]
            ended = [ids[i] for i in live if pos[i] + 1 == len(requests[i])]
            got = replay.step(entries, end=ended)
            for r, i in enumerate(live):
                check(got[r:r + 1], ref[i][pos[i]:pos[i] + 1], f"batch {batch} request {i} position {pos[i]}")
                pos[i] += 1
                if pos[i] == len(requests[i]):
                    del pos[i]
    return worst


@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", False), ("A", "bfloat16", False),
                                              ("B", "float32", False), ("B", "bfloat16", False),
                                              ("B", "float32", True), ("A", "bfloat16", True),
                                              ("C", "bfloat16", False), ("C", "float32", True),
                                              ("D", "bfloat16", False), ("D", "float32", False),
                                              ("E", "bfloat16", False), ("E", "float32", True)])
def test_every_cutting_gives_the_plain_logits(folders, plain_models, tmp_path, name, dtype, peaky):
    # The peaky variant of C is run in float32 only: with its head size and depth the bfloat16
    # rounding of the activations alone (whatever kernels compute the attention) moves the logits
    # by a tenth of their size, which says nothing about masks or cache addressing.
    storage = dtype                      # weights are stored in the precision that is tested
    folder = folders(name, storage, peaky)
    plain = plain_models(name, storage, peaky)
    requests = prompts_for(name, LENGTHS_C if name in ("C", "D") else LENGTHS)
    ref = [plain.logits(t) for t in requests]
    # the largest set of live requests is batch ([0,1,2]): 70 + 33 + 129 -> 128 + 64 + 192 tokens
    # (C: 170 + 33 + 257 -> 192 + 64 + 320)
    replay = Replay(folder, dtype, tmp_path, max_tokens=576 if name in ("C", "D") else 384)
    try:
        worst = run_all_cuttings(replay, requests, ref, dtype)
    finally:
        replay.close()
    print(f"tiny {name} {dtype} peaky={peaky}: largest error {worst:.3g}")


def test_replay_of_a_checkpoint_stored_in_bf16_run_in_float32(folders, plain_models, tmp_path):
    """float32 mode widens bf16 weights exactly, so it matches the plain model on the same file."""
    folder = folders("A", "bfloat16")
    plain = plain_models("A", "bfloat16")
    toks = prompts_for("A", [50])[0]
    replay = Replay(folder, "float32", tmp_path, max_tokens=64)
    try:
        got = replay.step([("x", toks, range(50))], end=["x"])
    finally:
        replay.close()
    ok, err, tol = close(got, plain.logits(toks), "float32")
    assert ok, (err, tol)


def test_replay_refuses_more_tokens_than_it_was_sized_for(folders, tmp_path):
    folder = folders("A", "float32")
    toks = prompts_for("A", [65])[0]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype",
                        "float32", "--out", str(tmp_path), "--max-tokens", "64"],
                       input=json.dumps({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [0]}], "end": []}) + "\n",
                       capture_output=True, text=True)
    assert p.returncode != 0 and "done 0" not in p.stdout
    assert "CacheFull" in p.stderr or "at most 64 tokens" in p.stderr


@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", True), ("B", "float32", False), ("B", "bfloat16", False),
                                              ("C", "float32", True), ("D", "bfloat16", False),
                                              ("E", "bfloat16", False), ("E", "float32", True)])
def test_prompts_cut_into_portions_and_requests_that_join_or_sit_out(folders, plain_models, tmp_path, name, dtype, peaky):
    """Steps that are neither whole prompts nor one token each: a request goes on by several tokens
    (portions of 2, portions that end on the 64-token page edge, portions longer than the window), sits
    out a step, or starts while others go on.  Same logits at every position as the plain model.
    (Tiny E with scaled queries and keys runs in float32 only: in bfloat16 the rounding of its activations alone
    moves the logits by 8 % of their size, in whole prompts as in portions, while float32 on the same weights is
    exact.)"""
    folder = folders(name, dtype, peaky)
    plain = plain_models(name, dtype, peaky)
    big = name in ("C", "D")
    requests = prompts_for(name, [257, 170, 45] if big else [129, 70, 45], seed=11)
    ref = [plain.logits(t) for t in requests]
    replay = Replay(folder, dtype, tmp_path, max_tokens=576 if big else 384)
    pos = [0, 0, 0]

    def step(*parts, end=()):
        """parts: (request, number of tokens); every position of every portion is checked."""
        entries = [(f"r{i}", requests[i][pos[i]:pos[i] + n], range(n)) for i, n in parts]
        got = replay.step(entries, end=[f"r{i}" for i in end])
        r = 0
        for i, n in parts:
            ok, err, tol = close(got[r:r + n], ref[i][pos[i]:pos[i] + n], dtype)
            assert ok, f"request {i} positions {pos[i]}..{pos[i] + n - 1}: error {err:.3g} > {tol:.3g}"
            pos[i] += n
            r += n
    try:
        a, b = len(requests[0]), len(requests[1])
        step((0, 2), (1, 62))                    # two start together
        step((0, 62))                            # request 1 sits out; request 0 reaches the page edge (64)
        step((0, 2), (1, 2), (2, 40))            # portions of 2 across the edge; request 2 joins the batch
        step((0, 1), (1, 1), (2, 1))             # an ordinary decode step in between
        step((0, a - 67 - 3), (2, 4), end=[2])   # a portion longer than every window; request 2 ends
        step((0, 3), (1, b - 65), end=[0, 1])
        assert pos == [a, b, 45]
        # what they held is free again: the longest request, whole
        got = replay.step([("again", requests[0], [a - 1])], end=["again"])
        ok, err, tol = close(got, ref[0][a - 1:a], dtype)
        assert ok, (err, tol)
    finally:
        replay.close()
