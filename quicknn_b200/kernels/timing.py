"""Single kernels timed alone, outside a model: the decode products and the prefill attention.

    python -m quicknn_b200.kernels.timing products  [--rows 8,16,32,64,128] [--model 2b|9b|27b]
    python -m quicknn_b200.kernels.timing attention [--tokens 2048,4096,8192] [--model 2b|9b|27b]

Every case is captured as a CUDA graph of ``--chain`` launches (26 by default, a model's depth) and the
graph is replayed five times between two CUDA events; the best replay divided by the chain is printed.
The products of a chain use a different weight matrix each, so that weights come from memory as they
do in a decode step and not from the L2 cache; programmatic dependent launch overlaps the launches as
it does in a step.  ``products`` prints, for each matrix of a layer, the time that reading the weights
once would take at the measured copy bandwidth, then the tcgen05 decode product, the mma.sync small-M
product (up to 64 rows) and ``torch.matmul`` (cuBLAS, for comparison only; no default path uses it).
``attention`` prints the tcgen05 kernel and the mma.sync kernel behind it with their TFLOP/s over the
causal triangle (4 x heads x head size x keys attended).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

LAYER_SIZES = {      # hidden, intermediate, heads, kv heads, head size, window
    "2b": (2304, 9216, 8, 4, 256, 4096),
    "9b": (3584, 14336, 16, 8, 256, 4096),
    "27b": (4608, 36864, 32, 16, 128, 4096),
}


def _copy_gbs() -> float:
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "..", "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6650.0


def _graph_time_us(torch, fn, chain: int, reps: int = 5) -> float:
    fn(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(chain):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(reps):
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / chain * 1e3)
    return best


def products(args) -> int:
    import torch
    from . import lib, ops
    dev, bf = "cuda:0", torch.bfloat16
    H, I, nq, nkv, hd, _ = LAYER_SIZES[args.model]
    shapes = {"q|k|v": ((nq + 2 * nkv) * hd, H, ops.EPI_NONE), "o": (H, nq * hd, ops.EPI_NONE),
              "gate|up": (2 * I, H, ops.EPI_GATED), "down": (H, I, ops.EPI_NONE)}
    L = lib.load()
    gbs = _copy_gbs()

    def small_m(x, w, epi):
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty((M, N // 2 if epi == ops.EPI_GATED else N), dtype=bf, device=dev)
        lib.check(L.qnn_skinny_bf16(ops._p(x), ops._p(w), ops._p(out), 1, M, N, K, epi, 0.0, 0, ops._stream()),
                  "qnn_skinny_bf16")
        return out

    print(f"layer sizes {args.model}; microseconds per product in a graph of {args.chain}; copy bandwidth {gbs:.0f} GB/s")
    print(f"{'rows':>5} {'matrix':8} {'weights once':>13} {'tcgen05':>9} {'mma.sync':>9} {'cuBLAS':>9}")
    for M in args.rows:
        for name, (N, K, epi) in shapes.items():
            W = [torch.randn(N, K, device=dev).to(bf) for _ in range(args.chain)]
            x = torch.randn(M, K, device=dev).to(bf)
            ideal = N * K * 2 / gbs / 1e3
            t_tc = _graph_time_us(torch, lambda i: ops.gemm_skinny_tcgen05(x, W[i], epilogue=epi), args.chain) \
                if M <= 128 else float("nan")
            t_mma = _graph_time_us(torch, lambda i: small_m(x, W[i], epi), args.chain) if M <= 64 else float("nan")
            t_lib = _graph_time_us(torch, lambda i: torch.matmul(x, W[i].t()), args.chain)
            print(f"{M:5d} {name:8} {ideal:13.1f} {t_tc:9.1f} {t_mma:9.1f} {t_lib:9.1f}")
            del W
    ops.raise_on_status(dev)
    return 0


def attention(args) -> int:
    import torch
    from . import ops
    dev = "cuda:0"
    _, _, nq, nkv, hd, window = LAYER_SIZES[args.model]
    cap = args.cap if args.cap > 0 else None
    keep = ops.ATTN_TCGEN05
    print(f"layer sizes {args.model}: {nq} heads of {hd} over {nkv} key/value heads, softcap {cap}; "
          f"microseconds per launch in a graph of {args.chain}")
    print(f"{'tokens':>7} {'prompts':>8} {'window':>7} {'tcgen05':>9} {'TFLOP/s':>9} {'mma.sync':>9} {'TFLOP/s':>9}")
    for T in args.tokens:
        for B, win in ((1, None), (args.prompts, None), (1, window)):
            if win is not None and T <= win:
                continue                                   # a window that nothing reaches is the first case again
            qkv = torch.randn(B * T, (nq + 2 * nkv) * hd, device=dev).to(torch.bfloat16)
            pos = torch.arange(T, device=dev, dtype=torch.int32).repeat(B)
            first = torch.arange(B, device=dev, dtype=torch.int32) * T
            row0 = first.repeat_interleave(T)
            lens = torch.full((B,), T, device=dev, dtype=torch.int32)
            keys = sum(min(p + 1, win) if win else p + 1 for p in range(T))
            flop = 4.0 * nq * hd * keys * B
            res = []
            for tensor_memory in (True, False):
                ops.ATTN_TCGEN05 = tensor_memory
                t = _graph_time_us(torch, lambda i: ops.attn_prefill(qkv, nq, nkv, hd, pos, row0, hd ** -0.5, cap, win,
                                                                     first, lens, T), args.chain)
                res += [t, flop / t / 1e6]
            print(f"{T:7d} {B:8d} {str(win):>7} {res[0]:9.1f} {res[1]:9.1f} {res[2]:9.1f} {res[3]:9.1f}")
    ops.ATTN_TCGEN05 = keep
    ops.raise_on_status(dev)
    return 0


def main(argv=None) -> int:
    ints = lambda s: [int(v) for v in s.split(",") if v]  # noqa: E731
    ap = argparse.ArgumentParser(prog="python -m quicknn_b200.kernels.timing", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    p = sub.add_parser("products", help="the four products of a layer at decode row counts")
    p.add_argument("--rows", type=ints, default=[8, 16, 32, 64, 128])
    a = sub.add_parser("attention", help="prefill attention over whole prompts")
    a.add_argument("--tokens", type=ints, default=[1024, 2048, 4096, 8192])
    a.add_argument("--prompts", type=int, default=8, help="the batched case: this many prompts of the same length")
    a.add_argument("--cap", type=float, default=50.0, help="softcap of the scores (0: none)")
    for q in (p, a):
        q.add_argument("--model", default="2b", choices=sorted(LAYER_SIZES))
        q.add_argument("--chain", type=int, default=26, help="launches per graph")
    args = ap.parse_args(argv)
    import torch
    if not torch.cuda.is_available():
        print("quicknn_b200.kernels.timing needs a CUDA device", file=sys.stderr)
        return 3
    return products(args) if args.what == "products" else attention(args)


if __name__ == "__main__":
    sys.exit(main())
