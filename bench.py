#!/usr/bin/env python3
"""Decode throughput of the Gemma 2 2B layer sizes on one B200, with prefill, roofline and
end-to-end figures on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

A "step" is one decode step of a batch of 8 sequences whose cached context reaches the
benchmark context length (8192) at the last timed step: from the ids that the step before chose
(greedy, on the device) to the ids of the next.  ``vs_baseline`` is against the same steps written
with plain PyTorch operations (``baseline/torch_ops_decode.py``): the reference publishes no
Gemma 2 figure and cannot run here.  Weights are random (seeded,
generated on the device); the cached history of the device-timed runs is random too
(``fill_synthetic``), because a decode step's time does not depend on the values.
Timing is by CUDA events on the launching stream after W warm-up steps; every step reads all
weights (5.2 GB) and the live cache, far more than the 126 MB L2, so no L2 flush is needed.
``e2e`` runs the same batch through the Python entry point (``LLM.generate``): prompts go in
as host lists, the prompts are really prefilled, and each step reads the sampled ids back.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Gemma 2 2B layer sizes
SIZES = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", hidden_size=2304, intermediate_size=9216,
    num_attention_heads=8, num_key_value_heads=4, head_dim=256, vocab_size=256000, num_hidden_layers=26,
    max_position_embeddings=8192, rope_theta=10000.0, rms_norm_eps=1e-6, sliding_window=4096,
    attn_logit_softcapping=50.0, final_logit_softcapping=30.0, query_pre_attn_scalar=256, eos_token_id=1,
    initializer_range=0.02)
# BASELINE.json configs[3] and configs[4]: the 9B and 27B layer sizes (only with --model)
OTHER_SIZES = {
    "9b": dict(hidden_size=3584, intermediate_size=14336, num_attention_heads=16, num_key_value_heads=8, head_dim=256,
               num_hidden_layers=42, query_pre_attn_scalar=256),
    "27b": dict(hidden_size=4608, intermediate_size=36864, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
                num_hidden_layers=46, query_pre_attn_scalar=144),
}
CONTEXT = 8192
BATCH = 8
PREFILL_TOKENS = 2048
RAMP_STEPS = 8
SEED = 2
FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS = 6650.0, 1590.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "source": "fallback"}
    try:
        with open(path) as fh:
            m = json.load(fh)
        if "hbm_gbs" in m:
            out["hbm_gbs"] = float(m["hbm_gbs"])
        if "bf16_tflops" in m:
            out["bf16_tflops"] = float(m["bf16_tflops"])
        out["source"] = "measured"
    except (OSError, ValueError, TypeError):
        pass
    return out


class Clocks:
    """Samples nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(int(float(r[0])))
                mx.append(int(float(r[1])))
            except (ValueError, IndexError):
                continue
            for name, v in zip(self.NAMES, r[2:]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi gave no samples"]}
        return {"sm_mhz": int(statistics.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def prefill_flops(cfg, T):
    """Products 2*T*K*N per matrix and causal attention 4*nq*hd*sum(keys seen), per layer, plus the head
    for one row."""
    H, I, nq, nkv, hd, L = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"],
                            cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"])
    mats = H * (nq + 2 * nkv) * hd + nq * hd * H + 3 * H * I
    total = 0
    for i in range(L):
        W = cfg["sliding_window"] if i % 2 == 0 else None
        keys = sum(min(p + 1, W) if W else p + 1 for p in range(T))
        total += 2 * T * mats + 4 * nq * hd * keys
    return total + 2 * H * cfg["vocab_size"]


def fill_synthetic(engine, slots, lengths, torch, seed=0):
    """Give sequences a history of the given lengths without computing it: pages are taken as a prompt
    of that length would take them and every cache line is filled with random keys and values.  For
    timing decode steps at a chosen context; the logits mean nothing."""
    engine.cache.extend(list(zip(slots, lengths)))
    engine.cache.sync()
    g = torch.Generator(device=engine.device)
    g.manual_seed(seed)
    for grp in engine.cache.groups:
        for t in (grp.k, grp.v):
            for li in range(t.shape[0]):
                t[li].normal_(0.0, 1.0, generator=g)


def timed_decode(engine, batch, steps, warmup, torch, with_clocks=False, context=CONTEXT, lengths=None, options=None):
    """Tokens per second of `steps` decode steps of `batch` sequences, each step from the ids that the
    step before chose on the device (greedy, or sampled with `options`) to the ids of the next.  The
    sequences end at `context` tokens, or start from the given `lengths`."""
    from quicknn_b200.sampling import GenerationOptions, Sampler
    vocab = engine.model.spec.embedding.vocab_size
    start = lengths if lengths is not None else [context - steps - warmup - RAMP_STEPS - 1] * batch
    slots = [engine.new_sequence() for _ in range(batch)]
    fill_synthetic(engine, slots, start, torch)
    sampler = Sampler(vocab, batch, options or GenerationOptions.greedy(1), engine.device)
    sampler.start(0, batch)
    tokens = torch.randint(1, vocab, (batch,), dtype=torch.int32, device=engine.device)
    tokens = engine.decode(slots, tokens, tail=sampler)          # eager pass, captures the graph
    for _ in range(warmup):
        tokens = engine.decode(slots, tokens, tail=sampler)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks = Clocks()
    ctx = clocks if with_clocks else open(os.devnull)
    with ctx:
        # untimed steps right before the timed ones, so that the SM clock that the sampler sees, and the
        # timed steps run at, is the clock under load (the device idles while nvidia-smi starts)
        for _ in range(RAMP_STEPS):
            tokens = engine.decode(slots, tokens, tail=sampler)
        torch.cuda.synchronize()
        k0 = engine.kernels_launched()
        e0.record()
        for _ in range(steps):
            tokens = engine.decode(slots, tokens, tail=sampler)
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = engine.kernels_launched() - k0
    sampler.read(tokens)                                        # raises if a step gave NaN or a kernel gave up
    bytes_step = engine.model.step_weight_bytes() + engine.cache.bytes_read_per_step(slots)
    for s in slots:
        engine.release(s)
    engine.forget_tail(sampler)
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "bytes_per_step": bytes_step,
            "launches": launches, "clocks": clocks.summary() if with_clocks else None}


def timed_baseline(cfg, steps, torch, context, batch):
    """The same decode steps and the same prefill with plain PyTorch operations (baseline/torch_ops_decode.py,
    tests/plain/gemma2_torch.py): bfloat16, cuBLAS products, a contiguous cache."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from torch_ops_decode import CachedTorchGemma2
    from plain.gemma2_torch import TorchGemma2
    from quicknn_b200.config.base import find_architecture
    from quicknn_b200.weights.random_init import random_tensors
    arch = find_architecture(cfg)
    weights = dict(random_tensors(arch, arch.config_cls.from_dict(cfg), SEED, torch.bfloat16, device="cuda:0"))
    steps = min(steps, 32)
    model = CachedTorchGemma2(cfg, weights, batch, context, "cuda:0", torch.bfloat16)
    model.fill_random(context - steps - 4)
    tokens = torch.randint(1, cfg["vocab_size"], (batch,), device="cuda:0")
    for _ in range(3):
        tokens = model.decode(tokens)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        tokens = model.decode(tokens)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    del model
    whole = TorchGemma2.from_tensors(cfg, weights, "cuda:0", torch.bfloat16)
    ids = torch.randint(1, cfg["vocab_size"], (PREFILL_TOKENS,)).tolist()
    times = []
    for i in range(5):
        torch.cuda.synchronize()
        e0.record()
        whole.logits(ids, [PREFILL_TOKENS - 1])
        e1.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(e0.elapsed_time(e1))
    del whole, weights
    torch.cuda.empty_cache()
    return {"impl": "plain PyTorch operations, bfloat16, cuBLAS products, contiguous cache", "value": round(batch / (ms / 1e3), 1),
            "unit": "tokens/s", "ms_per_step": round(ms, 3), "steps": steps,
            "prefill_ms": round(statistics.median(times), 3)}


def timed_tiny(torch):
    """BASELINE.json's two tiny workloads: the plain NumPy implementation on the CPU (whole sequence
    recomputed for every token) and this library in float32 on the GPU, seconds for all requests."""
    import tempfile
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import TINY, make_folder, prompts_for
    from plain.gemma2_plain import PlainGemma2
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, lens, new in (("A", [5, 11, 17], 8), ("B", [1, 6, 13, 29], 12)):
            folder = make_folder(tmp, name, "float32")
            prompts = prompts_for(name, lens)
            plain = PlainGemma2(folder, dtype=__import__("numpy").float32)
            t0 = time.perf_counter()
            ref = [plain.greedy(p, new) for p in prompts]
            out[f"{name.lower()}_plain_cpu_s"] = round(time.perf_counter() - t0, 4)
            llm = LLM(folder, max_context=64, max_batch=len(prompts), dtype="float32")
            llm.generate(prompts, GenerationOptions.greedy(new), stop_ids=[])       # warm-up: graphs, first launches
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            got = llm.generate(prompts, GenerationOptions.greedy(new), stop_ids=[])
            out[f"{name.lower()}_ours_s"] = round(time.perf_counter() - t0, 4)
            out[f"{name.lower()}_same_tokens"] = [r.tokens for r in got] == ref
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (reported in config)")
    ap.add_argument("--model", default="2b", choices=["2b", "9b", "27b"],
                    help="layer sizes; the record is for 2b (BASELINE.json configs[2])")
    ap.add_argument("--batch", type=int, default=BATCH, help="batch of the timed decode (the record is for 8)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context that the timed decode ends at")
    ap.add_argument("--no-graph", action="store_true", help="launch decode steps eagerly (for profilers)")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-baseline", action="store_true", help="do not time the plain PyTorch / NumPy baselines")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "HemulGM/QuickNN is Delphi-only Object Pascal (no setup.py/pyproject, pip cannot install "
                          "it; no Pascal compiler here) and its Gemma 2 path needs a Vulkan device: unavailable on "
                          "this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library is single-GPU by design (--gpus {args.gpus} refused)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions

    pk = peaks()
    base = dict(SIZES, **OTHER_SIZES.get(args.model, {}))
    if args.layers is None:
        args.layers = base["num_hidden_layers"]
    cfg = dict(base, num_hidden_layers=args.layers)
    # the large-batch point: 64 sequences, or the largest power of two whose cache fits beside the weights
    per_seq = sum(min(args.context, cfg["sliding_window"]) if i % 2 == 0 else args.context
                  for i in range(args.layers)) * cfg["num_key_value_heads"] * cfg["head_dim"] * 4
    weights = 2 * (cfg["vocab_size"] * cfg["hidden_size"] + args.layers * (
        cfg["hidden_size"] * (2 * cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
        + 3 * cfg["hidden_size"] * cfg["intermediate_size"]))
    big = 64
    while big > args.batch and big * per_seq + weights > 150e9:
        big //= 2
    max_b = max(big, args.batch) if not args.skip_points else args.batch
    llm = LLM.random(cfg, SEED, dtype="bfloat16", max_context=CONTEXT, max_batch=max_b,
                     max_tokens=max_b * CONTEXT)
    eng = llm.engine
    eng.use_graphs = not args.no_graph

    # ---- prefill of 2,048 tokens -----------------------------------------------------------
    # (first: its fraction is taken against the burst throughput of a GEMM, and after seconds of decoding the
    # GPU sits at its power cap, where the same prefill was measured 10 % slower)
    ids = torch.randint(1, cfg["vocab_size"], (PREFILL_TOKENS,)).tolist()
    times = []
    # 3 warm-ups, 3 timed, the median: prompts run back to back reach the power cap at about the sixth (8.05 -> 8.45 ms
    # here), and with an idle of 10 to 200 ms between them each meets a clock that is still rising (8.12 to 8.35 ms);
    # the fraction below is taken against the burst throughput of a product timed alone, so the prompts timed are
    # those of the burst state; ms_min and ms_max say what was seen
    for i in range(0 if args.skip_prefill else 6):
        slot = eng.new_sequence()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([(slot, ids)], "last")
        e1.record()
        torch.cuda.synchronize()
        eng.release(slot)
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    print(f"prefill ms: {[round(t, 3) for t in times]}", file=sys.stderr)
    pre_ms = statistics.median(times) if times else float("nan")
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    prefill = None if args.skip_prefill else {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
               # the timed steps run back to back: the last may already sit at the power cap
               "ms_min": round(min(times), 3), "ms_max": round(max(times), 3)}

    # ---- the headline: decode, batch 8 --------------------------------------------------
    main_run = timed_decode(eng, args.batch, args.steps, args.warmup, torch, with_clocks=True, context=args.context)
    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] / 1e3) / 1e9

    points, workload = {}, {}
    if not args.skip_points:
        for b in (1, big):
            points[f"decode_b{b}"] = round(timed_decode(eng, b, min(args.steps, 128), args.warmup, torch,
                                                        context=args.context)["tok_s"], 1)
        # the headline's steps with the reference's default sampling (temperature 0.6, top-k 20, top-p 0.95) instead
        # of the arg-max: the head writes its logits and the sampler's kernels run inside the step
        points[f"decode_b{args.batch}_sampled"] = round(timed_decode(
            eng, args.batch, min(args.steps, 128), args.warmup, torch, context=args.context,
            options=GenerationOptions(max_new_tokens=1))["tok_s"], 1)
        # BASELINE.json's workload as it is stated: prompts uniform in [512, 2048], then 256 decode steps
        import numpy as np
        rng = np.random.default_rng(SEED)
        for b in (1, BATCH, big):
            run = timed_decode(eng, b, 256, args.warmup, torch, lengths=rng.integers(512, 2049, b).tolist())
            workload[f"decode_b{b}"] = round(run["tok_s"], 1)
            workload[f"hbm_frac_b{b}"] = round(run["bytes_per_step"] / (run["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 3)
        # the workloads that are stated for the two larger sizes: 8 prompts uniform in [100, 6000] and 128 steps;
        # 16 prompts uniform in [256, 4096] and 64 steps
        stated = {"9b": (8, 100, 6000, 128), "27b": (16, 256, 4096, 64)}.get(args.model)
        if stated is not None and stated[0] <= max_b:
            n, lo, hi, steps_ = stated
            run = timed_decode(eng, n, steps_, args.warmup, torch, lengths=rng.integers(lo, hi + 1, n).tolist())
            workload[f"stated_b{n}_u{lo}_{hi}"] = round(run["tok_s"], 1)
            workload[f"stated_hbm_frac"] = round(run["bytes_per_step"] / (run["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 3)

    # ---- end to end through the Python entry point ------------------------------------------
    e2e = None
    if not args.skip_e2e:
        # as many steps as the device-timed run: the first 25 or so after the prompts run at a reduced SM clock
        # (the prefill of 8 x 8000 tokens hits the power cap; the clock takes about 80 ms to come back)
        # (so never fewer than 256 steps here, whatever the device-timed run was asked for)
        new = max(256, min(args.steps, 512))
        plen = CONTEXT - new - 1
        prompts = [torch.randint(1, cfg["vocab_size"], (plen,)).tolist() for _ in range(BATCH)]
        llm.max_batch = BATCH
        # a first call pays what is paid once (kernel attributes, the graphs of this sampler)
        llm.generate([p[:2048] for p in prompts], GenerationOptions.greedy(4), stop_ids=[])
        res = llm.generate(prompts, GenerationOptions.greedy(new), stop_ids=[])
        dec = max(r.decode_seconds for r in res)
        gen = sum(r.generated_tokens - 1 for r in res)
        ttft = max(r.time_to_first_token_seconds for r in res)
        e2e = {"value": round(gen / dec, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": round(llm.last_io["h2d_bytes_per_step"], 1),
               "d2h_bytes_per_step": round(llm.last_io["d2h_bytes_per_step"], 1), "steps": new, "prefill_seconds": round(ttft, 3),
               "prefill_tokens_per_s": round(BATCH * plen / ttft, 1)}

    # ---- the same steps with plain PyTorch operations; the tiny workloads with plain NumPy on the CPU --------
    baseline = tiny = None
    if not args.skip_baseline:
        del llm, eng
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        baseline = timed_baseline(cfg, args.steps, torch, args.context, args.batch)
        tiny = timed_tiny(torch)

    out = {
        "metric": f"decode tokens/s, Gemma 2 {args.model.upper()} layer sizes, batch {args.batch}, context {args.context}", "value": round(main_run["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(main_run["tok_s"] / baseline["value"], 2) if baseline else None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"gemma2-{args.model}-sizes", "global_batch": args.batch, "seq_len": args.context, "parallelism": "none",
                   "layers": args.layers, "layers_of_config": base["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "window": cfg["sliding_window"], "prefill_tokens": PREFILL_TOKENS, "weights": "random seed 2",
                   "l2": "each step reads > 5 GB, larger than L2; no flush", "peaks": pk["source"],
                   "step": "ids of one step to the ids of the next, greedy, on the device",
                   "baseline": "plain PyTorch ops bf16 (the reference publishes no figure)"},
        "clocks": main_run["clocks"], "gpu_launches": main_run["launches"],
        "e2e": e2e, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "workload_u512_2048": workload, "baseline": baseline, "tiny": tiny,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
