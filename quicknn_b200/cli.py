"""Command line.  Options are ``--name value``; ``--help`` lists them; an unknown option
is an error (the reference's argv style, Examples/Delphi/QwenImage21.dpr:46-107).  The
generation options carry the reference's names and defaults
(src/models/QuickNN.Models.LLM.Types.pas:144-155; MaxContext from
Examples/LLMChat/QuickNN.LLMChat.Settings.pas:38).

    python -m quicknn_b200 generate --model DIR --prompt-ids "5,17,3;9,4" --max-new-tokens 16 --temperature 0
    python -m quicknn_b200 random   --config config.json --seed 0 --out DIR
    python -m quicknn_b200 replay   --model DIR --dtype float32 --out DIR --max-tokens 4096 < trace.jsonl
    python -m quicknn_b200 info     --model DIR
    python -m quicknn_b200 chat     --model DIR          # a conversation over token ids: /new /memory /help /exit
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def _prompts(args) -> List[List[int]]:
    out: List[List[int]] = []
    if args.prompt_ids:
        for part in args.prompt_ids.split(";"):
            part = part.strip()
            if part:
                out.append([int(x) for x in part.replace(",", " ").split()])
    if args.prompt_file:
        with open(args.prompt_file, "r", encoding="utf-8") as fh:
            for line in fh:
                line = line.strip()
                if line:
                    ids = json.loads(line)
                    if isinstance(ids, dict):
                        ids = ids["tokens"]
                    out.append([int(x) for x in ids])
    if not out:
        raise SystemExit("generate: give --prompt-ids or --prompt-file")
    return out


def cmd_generate(args) -> int:
    from .engine import LLM
    from .sampling import GenerationOptions
    import torch
    if not torch.cuda.is_available():
        print("generate: no CUDA device; quicknn_b200 has no CPU path", file=sys.stderr)
        return 3
    prompts = _prompts(args)
    opts = GenerationOptions(max_new_tokens=args.max_new_tokens, hard_max_new_tokens=args.hard_max_new_tokens,
                             top_k=args.top_k, auto_continue=args.auto_continue, temperature=args.temperature,
                             top_p=args.top_p, repetition_penalty=args.repetition_penalty, seed=args.seed)
    opts.validate()
    llm = LLM(args.model, max_context=args.max_context, max_batch=args.max_batch, dtype=args.dtype,
              device=args.device)
    stops = None if args.stop_ids is None else [int(x) for x in args.stop_ids.replace(",", " ").split()]

    def on_token(i, tok):
        if args.stream:
            print(json.dumps({"request": i, "token": tok}), flush=True)

    def run():
        if not args.turns:
            return llm.generate(prompts, opts, on_token=on_token, stop_ids=stops)
        # the prompts are the turns of one conversation: each is appended to what was said so far, and only
        # what the cache does not hold yet is run
        out, said = [], []
        with llm.conversation() as chat:
            for i, turn in enumerate(prompts):
                r = chat.generate(said + turn, opts, on_token=lambda _, tok, i=i: on_token(i, tok), stop_ids=stops)
                r.index = i
                said = said + turn + r.tokens
                out.append(r)
        return out

    prof = None
    try:
        if args.profile:
            from .engine.profile import StepProfiler
            with StepProfiler(llm.engine) as prof:
                results = run()
        else:
            results = run()
    except KeyboardInterrupt:
        print("cancelled", file=sys.stderr)
        return 130
    for r in results:
        print(json.dumps({"request": r.index, "prompt_tokens": r.prompt_tokens, "tokens": r.tokens,
                          "finish_reason": r.finish_reason, "reused_tokens": r.reused_tokens,
                          "time_to_first_token_seconds": round(r.time_to_first_token_seconds, 6),
                          "decode_seconds": round(r.decode_seconds, 6),
                          "decode_tokens_per_second": round(r.decode_tokens_per_second(), 3)}))
    if prof is not None:
        print(prof.table(), file=sys.stderr)
    return 0


CHAT_HELP = ("/new: a new conversation, /memory: what the device holds, /help: this text, /exit: leave.  "
             "A line of token ids (\"5, 17, 3\") is a turn; Ctrl+C stops the reply that is being written; "
             "the history is cleared by /new only.")


class ChatSession:
    """The loop of the reference's chat console (Examples/LLMChat/QuickNNChat.dpr:126-205) over token ids instead
    of text: a line is a command or a turn; a turn is appended to what was said so far and answered, the answer's
    ids are written as they come, then a line of figures as the reference prints it (tokens, seconds, decode
    tokens per second, time to the first token, tokens said so far, tokens of the prompt found in the cache).  An
    error while answering drops the turn and starts the cache anew, as the reference does."""

    def __init__(self, llm, options, stop_ids, write, interrupted=lambda: False):
        self.llm, self.options, self.stop_ids = llm, options, stop_ids
        self.write, self.interrupted = write, interrupted
        self.chat = llm.conversation()
        self.said: List[int] = []

    def close(self) -> None:
        self.chat.close()

    def handle(self, line: str) -> bool:
        """One line of input; False when the session is over."""
        import time
        text = line.strip()
        if not text:
            return True
        command = text.lower()
        if command == "/exit":
            return False
        if command == "/help":
            self.write(CHAT_HELP + "\n")
            return True
        if command == "/memory":
            self.write(json.dumps(self.llm.memory_status()) + "\n")
            return True
        if command == "/new":
            self.chat.reset()
            self.said = []
            self.write("a new conversation\n")
            return True
        if text.startswith("/"):
            self.write(f"unknown command {text.split()[0]}; " + CHAT_HELP + "\n")
            return True
        try:
            turn = [int(x) for x in text.replace(",", " ").split()]
        except ValueError:
            self.write("a turn is a line of token ids, for instance: 5, 17, 3\n")
            return True
        start = time.perf_counter()
        try:
            r = self.chat.generate(self.said + turn, self.options, stop_ids=self.stop_ids,
                                   on_token=lambda _, tok: self.write(f"{tok} "), should_cancel=self.interrupted)
        except Exception as e:                       # the turn is dropped and the cache starts anew
            self.write(f"\n{type(e).__name__}: {e}\n")
            self.chat.reset()
            self.said = []
            return True
        self.said = self.said + turn + list(r.tokens)
        self.write(f"\n[{r.generated_tokens} tokens; {time.perf_counter() - start:.2f} s; decode: "
                   f"{r.decode_tokens_per_second():.1f} tokens/s; first token: {r.time_to_first_token_seconds:.3f} s; "
                   f"said so far: {len(self.said)}; reused: {r.reused_tokens}; {r.finish_reason}]\n")
        return True


def cmd_chat(args) -> int:
    import signal
    import torch
    from .engine import LLM
    from .sampling import GenerationOptions
    if not torch.cuda.is_available():
        print("chat: no CUDA device; quicknn_b200 has no CPU path", file=sys.stderr)
        return 3
    opts = GenerationOptions(max_new_tokens=args.max_new_tokens, hard_max_new_tokens=args.hard_max_new_tokens,
                             top_k=args.top_k, auto_continue=args.auto_continue, temperature=args.temperature,
                             top_p=args.top_p, repetition_penalty=args.repetition_penalty, seed=args.seed)
    opts.validate()
    llm = LLM(args.model, max_context=args.max_context, max_batch=1, dtype=args.dtype, device=args.device)
    stops = None if args.stop_ids is None else [int(x) for x in args.stop_ids.replace(",", " ").split()]
    state = {"interrupted": False}

    def write(text: str) -> None:
        sys.stdout.write(text)
        sys.stdout.flush()

    status = llm.memory_status()
    write(f"model: {args.model}\ncache: {status['cache_bytes'] / 1048576.0:.1f} MiB; context: {args.max_context} tokens\n")
    write(CHAT_HELP + "\n")
    session = ChatSession(llm, opts, stops, write, lambda: state["interrupted"])
    previous = signal.signal(signal.SIGINT, lambda *_: state.__setitem__("interrupted", True))
    try:
        while True:
            state["interrupted"] = False
            write("> ")
            line = sys.stdin.readline()
            if not line or not session.handle(line):
                break
    finally:
        signal.signal(signal.SIGINT, previous)
        session.close()
    return 0


def cmd_random(args) -> int:
    import torch
    from .config.base import find_architecture
    from .weights import write_model_folder
    with open(args.config, "r", encoding="utf-8") as fh:
        raw = json.load(fh)
    arch = find_architecture(raw)
    cfg = arch.config_cls.from_dict(raw)
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    write_model_folder(args.out, arch, cfg, args.seed, dt, args.norm_std)
    print(args.out)
    return 0


def cmd_info(args) -> int:
    from .config.base import load_config
    from .parts import expected_tensors
    arch, cfg = load_config(args.model)
    spec = arch.build_spec(cfg)
    tensors = expected_tensors(spec)
    n = 0
    for shape, _ in tensors.values():
        c = 1
        for d in shape:
            c *= d
        n += c
    print(json.dumps({"architecture": arch.name, "layers": len(spec.layers), "tensors": len(tensors),
                      "parameters": n, "config": cfg.to_dict()}, indent=1))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="quicknn_b200", description=__doc__.split("\n")[0], allow_abbrev=False)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids for prompts given as token ids", allow_abbrev=False)
    g.add_argument("--model", required=True)
    g.add_argument("--prompt-ids", help='prompts as ids, ";" between prompts: "5,17,3;9,4"')
    g.add_argument("--prompt-file", help="one JSON list of ids (or {\"tokens\": [...]}) per line")
    g.add_argument("--max-new-tokens", type=int, default=256)
    g.add_argument("--hard-max-new-tokens", type=int, default=4096)
    g.add_argument("--auto-continue", action="store_true")
    g.add_argument("--top-k", type=int, default=20)
    g.add_argument("--temperature", type=float, default=0.6)
    g.add_argument("--top-p", type=float, default=0.95)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=42)
    g.add_argument("--stop-ids", default=None, help="override the configuration's eos_token_id")
    g.add_argument("--max-context", type=int, default=2048)
    g.add_argument("--max-batch", type=int, default=8)
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--stream", action="store_true", help="print each token as it is produced")
    g.add_argument("--turns", action="store_true",
                   help="the prompts are successive turns of one conversation that keeps its cache (reused_tokens "
                        "says how much of each turn's prompt was found there)")
    g.add_argument("--profile", action="store_true",
                   help="time every step and every kind of part with CUDA events (steps then run eagerly) and print a table")
    g.set_defaults(fn=cmd_generate)

    c = sub.add_parser("chat", help="a conversation over token ids, read line by line: /new /memory /help /exit",
                       allow_abbrev=False)
    c.add_argument("--model", required=True)
    c.add_argument("--max-new-tokens", type=int, default=256)
    c.add_argument("--hard-max-new-tokens", type=int, default=4096)
    c.add_argument("--auto-continue", action="store_true")
    c.add_argument("--top-k", type=int, default=20)
    c.add_argument("--temperature", type=float, default=0.6)
    c.add_argument("--top-p", type=float, default=0.95)
    c.add_argument("--repetition-penalty", type=float, default=1.0)
    c.add_argument("--seed", type=int, default=42)
    c.add_argument("--stop-ids", default=None, help="override the configuration's eos_token_id")
    c.add_argument("--max-context", type=int, default=2048)
    c.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    c.add_argument("--device", default="cuda:0")
    c.set_defaults(fn=cmd_chat)

    r = sub.add_parser("random", help="write a model folder with random weights", allow_abbrev=False)
    r.add_argument("--config", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    r.add_argument("--norm-std", type=float, default=None)
    r.set_defaults(fn=cmd_random)

    i = sub.add_parser("info", help="print what a model folder's configuration describes", allow_abbrev=False)
    i.add_argument("--model", required=True)
    i.set_defaults(fn=cmd_info)

    p = sub.add_parser("replay", help="trace replay (same as bin/trace_run)", add_help=False)
    p.set_defaults(fn=None)

    argv = sys.argv[1:] if argv is None else list(argv)
    if argv and argv[0] == "replay":
        from .replay import main as replay_main
        return replay_main(argv[1:])
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
