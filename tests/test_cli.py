"""The command line: ``python -m quicknn_b200 random | info | generate`` and its refusals."""
import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT, TINY, prompts_for


def run(*argv, stdin=None):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run([sys.executable, "-m", "quicknn_b200", *argv], input=stdin, capture_output=True, text=True,
                          env=env, cwd=str(ROOT))


def test_random_writes_a_folder_that_info_describes(tmp_path):
    raw, seed, _ = TINY["B"]
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(raw))
    out = tmp_path / "model"
    p = run("random", "--config", str(cfg), "--seed", str(seed), "--out", str(out), "--dtype", "float32")
    assert p.returncode == 0, p.stderr
    assert p.stdout.strip() == str(out)
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    p = run("info", "--model", str(out))
    assert p.returncode == 0, p.stderr
    info = json.loads(p.stdout)
    H, I, V, L = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"], raw["num_hidden_layers"]
    nq, nkv, hd = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
    per_layer = H * (nq + 2 * nkv) * hd + nq * hd * H + 3 * H * I + 4 * H
    assert info["architecture"] == "Gemma2ForCausalLM" and info["layers"] == L
    assert info["parameters"] == V * H + L * per_layer + H
    assert info["config"]["sliding_window"] == raw["sliding_window"]
    # the same seed gives the same file; another seed another
    out2 = tmp_path / "again"
    assert run("random", "--config", str(cfg), "--seed", str(seed), "--out", str(out2), "--dtype", "float32").returncode == 0
    assert (out / "model.safetensors").read_bytes() == (out2 / "model.safetensors").read_bytes()


def test_unknown_options_and_commands_are_errors(tmp_path):
    p = run("info", "--model", str(tmp_path), "--verbose")
    assert p.returncode == 2 and "unrecognized arguments" in p.stderr
    p = run("info", "--mod", str(tmp_path))             # no abbreviations
    assert p.returncode == 2
    p = run("serve")
    assert p.returncode == 2 and "invalid choice" in p.stderr
    p = run("generate", "--model", str(tmp_path), "--top-k", "many")
    assert p.returncode == 2
    p = run("--help")
    assert p.returncode == 0 and "generate" in p.stdout and "random" in p.stdout


def test_generate_without_a_gpu_says_so_in_one_line(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this machine has a CUDA device")
    p = run("generate", "--model", str(tmp_path), "--prompt-ids", "5,6")
    assert p.returncode == 3 and "Traceback" not in p.stderr and "no CUDA device" in p.stderr


@pytest.mark.gpu
def test_generate_prints_what_the_plain_model_generates(folders, plain_models, tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    folder = folders("A", "float32")
    plain = plain_models("A", "float32")
    prompts = prompts_for("A", [5, 11, 17])
    ids = ";".join(",".join(str(t) for t in p) for p in prompts)
    p = run("generate", "--model", folder, "--prompt-ids", ids, "--max-new-tokens", "8", "--temperature", "0",
            "--dtype", "float32", "--max-context", "64", "--stop-ids", "", "--stream")
    assert p.returncode == 0, p.stderr
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.strip()]
    results = [l for l in lines if "tokens" in l]
    streamed = [l for l in lines if "token" in l]
    assert len(results) == 3 and len(streamed) == 24
    for r, pr in zip(results, prompts):
        assert r["tokens"] == plain.greedy(pr, 8) and r["finish_reason"] == "max_tokens"
        assert [s["token"] for s in streamed if s["request"] == r["request"]] == r["tokens"]
    # prompts from a file, a stop id, and an option that the options' own rules refuse
    f = tmp_path / "prompts.jsonl"
    f.write_text(json.dumps(prompts[0]) + "\n" + json.dumps({"tokens": prompts[1]}) + "\n")
    stop = plain.greedy(prompts[1], 8)[3]
    p = run("generate", "--model", folder, "--prompt-file", str(f), "--max-new-tokens", "8", "--temperature", "0",
            "--dtype", "float32", "--max-context", "64", "--stop-ids", str(stop))
    assert p.returncode == 0, p.stderr
    got = [json.loads(l) for l in p.stdout.splitlines() if l.strip()]
    assert got[1]["tokens"] == plain.greedy(prompts[1], 8, stop_ids=[stop]) and got[1]["finish_reason"] == "eos"
    p = run("generate", "--model", folder, "--prompt-ids", "5", "--top-p", "1.5")
    assert p.returncode != 0
    # the same prompts as the turns of one conversation: each reply is the plain model's for everything said so far
    p = run("generate", "--model", folder, "--prompt-ids", ids, "--max-new-tokens", "4", "--temperature", "0",
            "--dtype", "float32", "--max-context", "128", "--stop-ids", "", "--turns")
    assert p.returncode == 0, p.stderr
    got = [json.loads(l) for l in p.stdout.splitlines() if l.strip()]
    said = []
    for r, turn in zip(got, prompts):
        assert r["tokens"] == plain.greedy(said + turn, 4)
        assert r["reused_tokens"] in (max(0, len(said) - 1), len(said))       # all that was said, but for a reply's last token
        said = said + turn + r["tokens"]



class _FakeConversation:
    def __init__(self, log):
        self.log, self.held = log, []

    def reset(self):
        self.log.append("reset")
        self.held = []

    def close(self):
        self.log.append("close")

    def generate(self, prompt, options, on_token=None, stop_ids=None, should_cancel=None):
        from quicknn_b200.engine.generate import GenerationResult
        if prompt[-1] == 666:
            raise RuntimeError("the device said no")
        reused = 0
        while reused < min(len(self.held), len(prompt) - 1) and self.held[reused] == prompt[reused]:
            reused += 1
        r = GenerationResult(index=0, prompt_tokens=len(prompt))
        for t in (prompt[-1] + 1, prompt[-1] + 2):
            if should_cancel is not None and should_cancel():
                break
            r.tokens.append(t)
            on_token(0, t)
        r.finish_reason = "max_tokens"
        r.reused_tokens = reused
        self.held = list(prompt) + r.tokens
        self.log.append(("generate", list(prompt), stop_ids))
        return r


class _FakeLLM:
    def __init__(self):
        self.log = []

    def conversation(self):
        return _FakeConversation(self.log)

    def memory_status(self):
        return {"weight_bytes": 10, "cache_bytes": 20}


def test_the_chat_loop_takes_commands_and_turns():
    """``chat`` without a model: commands, turns that carry the history, an error that drops the turn and
    starts anew, a reply that is interrupted, the figures after a reply."""
    from quicknn_b200.cli import CHAT_HELP, ChatSession
    out, stop = [], {"now": False}
    llm = _FakeLLM()
    s = ChatSession(llm, None, [1], out.append, lambda: stop["now"])
    assert s.handle("\n") and s.handle("/help\n") and out[-1].startswith(CHAT_HELP)
    assert s.handle("/memory") and json.loads(out[-1]) == {"weight_bytes": 10, "cache_bytes": 20}
    assert s.handle("/nonsense") and out[-1].startswith("unknown command /nonsense")
    assert s.handle("five six") and "token ids" in out[-1]
    assert llm.log == []
    out.clear()
    assert s.handle("5, 17 3\n")
    assert llm.log[-1] == ("generate", [5, 17, 3], [1])
    assert out[:2] == ["4 ", "5 "] and "[2 tokens;" in out[-1] and "reused: 0; max_tokens]" in out[-1]
    assert s.handle("9")                                                   # the next turn carries what was said
    assert llm.log[-1] == ("generate", [5, 17, 3, 4, 5, 9], [1]) and "said so far: 8; reused: 5;" in out[-1]
    assert s.handle("666") and "RuntimeError: the device said no" in out[-1] and llm.log[-1] == "reset"
    assert s.handle("7") and llm.log[-1] == ("generate", [7], [1])         # the history went with the failed turn
    assert s.handle("/NEW") and llm.log[-1] == "reset" and out[-1] == "a new conversation\n"
    stop["now"] = True
    out.clear()
    assert s.handle("3") and "[0 tokens;" in out[-1]                         # interrupted before the first token
    assert not s.handle(" /exit ")
    s.close()
    assert llm.log[-1] == "close"


@pytest.mark.gpu
def test_chat_answers_turns_as_the_plain_model_does(folders, plain_models):
    """``chat`` on a tiny model, its lines from standard input: two turns of one conversation, /memory, /new, the
    first turn again (the same reply), /exit; every reply is the plain model's for everything said so far."""
    import re
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    folder = folders("A", "float32")
    plain = plain_models("A", "float32")
    first, second = prompts_for("A", [6, 3], seed=8)
    lines = [", ".join(map(str, first)), " ".join(map(str, second)), "/memory", "/new", ",".join(map(str, first)), "/exit",
             "5, 5"]
    p = run("chat", "--model", folder, "--max-new-tokens", "5", "--temperature", "0", "--dtype", "float32",
            "--max-context", "64", "--stop-ids", "", stdin="\n".join(lines) + "\n")
    assert p.returncode == 0, p.stderr
    replies = re.findall(r"> ((?:\d+ )+)\n\[(\d+) tokens; .*?reused: (\d+); (\w+)\]", p.stdout)
    assert len(replies) == 3, p.stdout
    a = plain.greedy(first, 5)
    b = plain.greedy(first + a + second, 5)
    assert [int(t) for t in replies[0][0].split()] == a and replies[0][1:] == ("5", "0", "max_tokens")
    assert [int(t) for t in replies[1][0].split()] == b and int(replies[1][2]) >= len(first) + len(a) - 1
    assert [int(t) for t in replies[2][0].split()] == a and replies[2][2] == "0"       # /new forgot the history
    assert '"cache_bytes"' in p.stdout and "a new conversation" in p.stdout
    assert p.stdout.count("> ") == 6                                                  # six lines are read, none after /exit
