"""Each part alone against the plain functions, and a toy mixer with state of its own that is
registered, built and stepped without a change to the library's files."""
import dataclasses
import json
import math
import os

import numpy as np
import pytest
import torch

from plain import gemma2_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.asarray(a)).to(DEV).to(dtype).contiguous()


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rnd(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).normal(size=shape) * scale).astype(np.float32)


def make_step(lens, starts, slots, mode, dtype, cache, splits=2, part=None):
    from quicknn_b200.engine.batch import StepBatch
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)  # noqa: E731
    T = sum(lens)
    pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lens)])
    slot = np.concatenate([np.full(n, s) for s, n in zip(slots, lens)])
    row0 = np.concatenate([np.full(n, r) for r, n in zip(np.cumsum([0] + lens[:-1]), lens)])
    cache.extend([(s, st + n) for s, st, n in zip(slots, starts, lens)])
    cache.sync()
    step = StepBatch(mode, T, len(lens), i32(np.zeros(T)), i32(pos), i32(slot), i32(row0), i32(slots), i32([T - 1]),
                     dtype, max(lens), max_seq=cache.max_seq, tuning={"decode_splits": splits})
    need = part.scratch_need(step) if part is not None else 0      # what the engine does for all parts of a model
    step.scratch = torch.empty(need, dtype=torch.uint8, device=DEV) if need else None
    return step


def test_norm_part():
    from quicknn_b200.parts import NORMS, PartSpec
    spec = PartSpec("rmsnorm", {"size": 100, "eps": 1e-5, "unit_offset": True})
    cls = NORMS.get("rmsnorm")
    assert cls.param_shapes(spec) == {"weight": ((100,), "norm")}
    n = cls(spec)
    w, x = rnd(100, 1, 0.2), rnd((4, 100), 2, 3.0)
    n.load({"weight": dev(w)}, torch.float32, DEV)
    assert np.abs(host(n(dev(x), torch.float32)) - P.rmsnorm(x.astype(np.float64), w, 1e-5)).max() < 1e-5
    plain_w = cls(PartSpec("rmsnorm", {"size": 100, "eps": 1e-5}))           # the "w" flavour
    plain_w.load({"weight": dev(w)}, torch.float32, DEV)
    assert np.abs(host(plain_w(dev(x), torch.float32)) - P.rmsnorm(x.astype(np.float64), w - 1, 1e-5)).max() < 1e-5


def test_rotary_part_tables():
    from quicknn_b200.parts import POSITIONS, PartSpec
    r = POSITIONS.get("rotary")(PartSpec("rotary", {"head_dim": 24, "theta": 1e6, "rotary_dim": 24}))
    r.prepare(DEV)
    j = np.arange(12)
    assert np.array_equal(host(r.inv_freq), np.exp(-math.log(1e6) * 2 * j / 24).astype(np.float32).astype(np.float64))
    with pytest.raises(ValueError):
        POSITIONS.get("rotary")(PartSpec("rotary", {"head_dim": 24, "theta": 1e4, "rotary_dim": 30}))
    none = POSITIONS.get("none")(PartSpec("none", {}))
    none.prepare(DEV)
    assert none.rotary_dim == 0 and none.inv_freq.numel() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_mlp_part(dtype):
    from quicknn_b200.parts import FEED_FORWARDS, PartSpec
    spec = PartSpec("gated_mlp", {"hidden_size": 96, "intermediate_size": 200, "activation": "gelu_tanh"})
    cls = FEED_FORWARDS.get("gated_mlp")
    assert cls.param_shapes(spec)["down_proj"] == ((96, 200), "matrix")
    ff = cls(spec)
    bf = lambda a: torch.from_numpy(a).to(torch.bfloat16).float().numpy()  # noqa: E731
    wg, wu, wd = bf(rnd((200, 96), 1, 0.1)), bf(rnd((200, 96), 2, 0.1)), bf(rnd((96, 200), 3, 0.1))
    ff.load({"gate_proj": dev(wg, dtype), "up_proj": dev(wu, dtype), "down_proj": dev(wd, dtype)}, dtype, DEV)
    for rows in (3, 70):                      # the small-M kernels and the whole-prompt path
        x = bf(rnd((rows, 96), 4 + rows))
        got = host(ff.forward(dev(x, dtype), None))
        ref = P.geglu_mlp(x.astype(np.float64), wg, wu, wd)
        assert np.abs(got - ref).max() < (1e-5 if dtype == torch.float32 else 0.03) * max(1, np.abs(ref).max())
    with pytest.raises(ValueError):
        cls(PartSpec("gated_mlp", {"hidden_size": 8, "intermediate_size": 8, "activation": "relu"}))


@pytest.mark.parametrize("window", [None, 5])
def test_attention_part_prefill_then_decode(window):
    """The mixer alone over a cache of its own: two prompts in one step, then tokens one by one,
    against plain projections + rotation + attention over the whole sequence."""
    from quicknn_b200.cache import KVCache
    from quicknn_b200.parts import MIXERS, PartSpec
    H, nq, nkv, hd = 48, 6, 2, 24
    pos_spec = PartSpec("rotary", {"head_dim": hd, "theta": 1e4, "rotary_dim": hd})
    spec = PartSpec("attention", {"hidden_size": H, "n_heads": nq, "n_kv_heads": nkv, "head_dim": hd,
                                  "scale": 0.2, "softcap": 20.0, "window": window, "position": pos_spec})
    mixer = MIXERS.get("attention")(spec)
    assert mixer.cache_need().window == window and mixer.state_need() is None
    w = {"q_proj": rnd((nq * hd, H), 1, 0.3), "k_proj": rnd((nkv * hd, H), 2, 0.3),
         "v_proj": rnd((nkv * hd, H), 3, 0.3), "o_proj": rnd((H, nq * hd), 4, 0.3)}
    mixer.load({k: dev(v) for k, v in w.items()}, torch.float32, DEV)
    cache = KVCache([mixer.cache_need()], [None], 512, 3, 256, torch.float32, DEV)
    lens = [70, 9]
    xs = [rnd((n + 6, H), 10 + i) for i, n in enumerate(lens)]

    def plain(x):
        T = x.shape[0]
        x = x.astype(np.float64)
        q = P.rope((x @ w["q_proj"].T).reshape(T, nq, hd), np.arange(T), 1e4)
        k = P.rope((x @ w["k_proj"].T).reshape(T, nkv, hd), np.arange(T), 1e4)
        v = (x @ w["v_proj"].T).reshape(T, nkv, hd)
        return P.attention(q, k, v, 0.2, 20.0, window).reshape(T, -1) @ w["o_proj"].T
    ref = [plain(x) for x in xs]
    slots = [cache.allocate(), cache.allocate()]
    slots = slots[::-1]
    step = make_step(lens, [0, 0], slots, "prefill", torch.float32, cache, part=mixer)
    assert step.scratch is None                                    # prompts need no scratch
    y = host(mixer.forward(dev(np.concatenate([x[:n] for x, n in zip(xs, lens)])), step, cache.line(0)))
    assert np.abs(y - np.concatenate([r[:n] for r, n in zip(ref, lens)])).max() < 2e-5
    for t in range(6):
        step = make_step([1, 1], [n + t for n in lens], slots, "decode", torch.float32, cache, part=mixer)
        ranges = mixer.decode_splits(step)
        assert ranges > 1 and step.scratch.numel() == 2 * nq * ranges * (hd + 2) * 4    # rows x heads x ranges x (head + 2) floats
        y = host(mixer.forward(dev(np.stack([x[n + t] for x, n in zip(xs, lens)])), step, cache.line(0)))
        assert np.abs(y - np.stack([r[n + t] for r, n in zip(ref, lens)])).max() < 2e-5


def test_sandwich_block_against_the_plain_layer(folders, plain_models):
    """One whole layer of tiny B from its own tensors."""
    from quicknn_b200.cache import KVCache
    from quicknn_b200.config import Gemma2Config, gemma2_spec
    from quicknn_b200.parts import BLOCKS
    from conftest import TINY_B
    plain = plain_models("B")
    spec = gemma2_spec(Gemma2Config.from_dict(TINY_B))
    layer = spec.layers[1]
    blk = BLOCKS.get("sandwich")(layer)
    blk.load({ln: dev(plain.w[cn]) for ln, cn in layer.tensors.items()}, torch.float32, DEV)
    cache = KVCache([blk.mixer.cache_need()], [None], 128, 1, 128, torch.float32, DEV)
    slot = cache.allocate()
    T = 21
    x = rnd((T, 96), 7)
    step = make_step([T], [0], [slot], "prefill", torch.float32, cache)
    resid = dev(x)
    blk.forward(resid, step, cache.line(0))
    w, p, xx = plain.w, "model.layers.1.", x.astype(np.float64)
    n = P.rmsnorm(xx, w[p + "input_layernorm.weight"], plain.eps)
    q = P.rope((n @ w[p + "self_attn.q_proj.weight"].T).reshape(T, 6, 24), np.arange(T), plain.theta)
    k = P.rope((n @ w[p + "self_attn.k_proj.weight"].T).reshape(T, 1, 24), np.arange(T), plain.theta)
    v = (n @ w[p + "self_attn.v_proj.weight"].T).reshape(T, 1, 24)
    a = P.attention(q, k, v, plain.scale, plain.attn_cap, None).reshape(T, -1) @ w[p + "self_attn.o_proj.weight"].T
    xx = xx + P.rmsnorm(a, w[p + "post_attention_layernorm.weight"], plain.eps)
    n = P.rmsnorm(xx, w[p + "pre_feedforward_layernorm.weight"], plain.eps)
    y = P.geglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    xx = xx + P.rmsnorm(y, w[p + "post_feedforward_layernorm.weight"], plain.eps)
    assert np.abs(host(resid) - xx).max() < 2e-5 * max(1.0, np.abs(xx).max())


# ---- a toy architecture, defined here, with a mixer that keeps state of its own -------------

def _define_toy():
    from quicknn_b200.config.base import (Architecture, ModelConfig, as_float, as_int, register_architecture)
    from quicknn_b200.kernels import ops
    from quicknn_b200.parts import (MIXERS, EmbeddingSpec, HeadSpec, LayerSpec, Mixer, ModelSpec, PartSpec,
                                    ScheduleEntry, StateNeed)

    @MIXERS.register("toy_decay", replace=True)
    class DecayMixer(Mixer):
        """y_t = W s_t with the per-sequence state s_t = decay * s_{t-1} + x_t: no keys, no
        values, a state of fixed size that lives in the cache's state region."""

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden, self.decay = int(spec.params["hidden_size"]), float(spec.params["decay"])

        @classmethod
        def param_shapes(cls, spec):
            h = int(spec.params["hidden_size"])
            return {"mix": ((h, h), cls.PARAM_ROLE_MATRIX)}

        def load(self, tensors, compute_dtype, device):
            self.w = tensors["mix"].contiguous()

        def weight_bytes(self):
            return self.w.numel() * self.w.element_size()

        def state_need(self):
            return StateNeed((self.hidden,), "float32")

        def scratch_need(self, step):
            return step.n_tokens * self.hidden * 4          # the running sums of the step's rows, float32

        def forward(self, x, step, line):
            slots = step.tok_slot.cpu().tolist()
            xf = x.float()
            assert step.scratch is not None and step.scratch.numel() >= self.scratch_need(step)
            out = step.scratch[:xf.numel() * 4].view(torch.float32).view(xf.shape)
            for t, s in enumerate(slots):                   # a toy: token by token
                if s < 0:
                    out[t] = 0
                    continue
                line.state[s].mul_(self.decay).add_(xf[t])
                out[t] = line.state[s]
            return ops.linear(out.to(x.dtype).contiguous(), self.w)

    def _f(conv, **kw):
        return dataclasses.field(default=kw.get("default"), metadata={"convert": conv, "required": "default" not in kw})

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden_size: int = _f(as_int)
        vocab_size: int = _f(as_int)
        n_heads: int = _f(as_int)
        head_dim: int = _f(as_int)
        inner: int = _f(as_int)
        decay: float = _f(as_float)
        eps: float = _f(as_float)
        max_position_embeddings: int = _f(as_int)

    def toy_spec(c):
        H = c.hidden_size
        norm = PartSpec("rmsnorm", {"size": H, "eps": c.eps, "unit_offset": False})
        ff = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": c.inner, "activation": "silu"})
        attn = PartSpec("attention", {"hidden_size": H, "n_heads": c.n_heads, "n_kv_heads": c.n_heads,
                                      "head_dim": c.head_dim, "scale": c.head_dim ** -0.5, "softcap": None,
                                      "window": None, "position": PartSpec("none", {})})
        toy = PartSpec("toy_decay", {"hidden_size": H, "decay": c.decay})

        def layer(i, mixer, names):
            t = {f"ff.{n}_proj": f"l{i}.{n}" for n in ("gate", "up", "down")}
            t.update({"norms.pre_mixer.weight": f"l{i}.n1", "norms.pre_ff.weight": f"l{i}.n2"})
            t.update({f"mixer.{k}": f"l{i}.{v}" for k, v in names.items()})
            return LayerSpec(PartSpec("prenorm", {}), mixer, ff, {"pre_mixer": norm, "pre_ff": norm}, t)
        layers = (layer(0, toy, {"mix": "mix"}),
                  layer(1, attn, {f"{x}_proj": x for x in "qkvo"}))
        # the order of execution is data: layer 0 runs twice (each run with a state line of its own),
        # and the last entry runs layer 1's weights again on the cache line that its first run wrote
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(1, 1, writes_cache=False))
        return ModelSpec("ToyForTest", H, EmbeddingSpec(c.vocab_size, H, 1.0, "emb"), layers, schedule,
                         HeadSpec(c.vocab_size, H, True, None, None, norm, "nf"), c.max_position_embeddings,
                         init_std=0.3, init_norm_std=0.2)

    arch = register_architecture(Architecture("ToyForTest", ToyConfig, toy_spec), replace=True)
    return arch, ToyConfig


def _toy_plain(w, cfg, ids):
    """The toy model in NumPy, whole sequence."""
    H, nh, hd = cfg["hidden_size"], cfg["n_heads"], cfg["head_dim"]
    norm = lambda x, g: x / np.sqrt((x * x).mean(-1, keepdims=True) + cfg["eps"]) * g  # noqa: E731
    silu = lambda x: x / (1 + np.exp(-x))  # noqa: E731
    x = w["emb"][ids].astype(np.float64)
    T = len(ids)

    def ff(i, x):
        n = norm(x, w[f"l{i}.n2"])
        return x + (silu(n @ w[f"l{i}.gate"].T) * (n @ w[f"l{i}.up"].T)) @ w[f"l{i}.down"].T

    def decay(x):
        n = norm(x, w["l0.n1"])
        s, out = np.zeros(H), np.zeros_like(n)
        for t in range(T):
            s = cfg["decay"] * s + n[t]
            out[t] = s
        return ff(0, x + out @ w["l0.mix"].T)

    kv = {}

    def attn(x, reuse):
        n = norm(x, w["l1.n1"])
        q = (n @ w["l1.q"].T).reshape(T, nh, hd)
        if not reuse:
            kv["k"], kv["v"] = (n @ w["l1.k"].T).reshape(T, nh, hd), (n @ w["l1.v"].T).reshape(T, nh, hd)
        a = P.attention(q, kv["k"], kv["v"], hd ** -0.5, None, None).reshape(T, -1)
        return ff(1, x + a @ w["l1.o"].T)
    x = attn(decay(attn(decay(x), False)), True)
    return norm(x, w["nf"]) @ w["emb"].T


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    from quicknn_b200.engine import Engine, Model
    from quicknn_b200.weights import write_model_folder
    arch, ToyConfig = _define_toy()
    raw = dict(architectures=["ToyForTest"], hidden_size=40, vocab_size=90, n_heads=2, head_dim=16, inner=56,
               decay=0.7, eps=1e-5, max_position_embeddings=256)
    cfg = ToyConfig.from_dict(raw)
    folder = write_model_folder(str(tmp_path / "toy"), arch, cfg, 5, torch.float32)
    with open(os.path.join(folder, "config.json")) as fh:
        assert json.load(fh)["decay"] == 0.7
    model = Model.from_folder(folder, "float32", DEV)            # found through the registry by name
    needs, states = model.cache_needs()
    assert [n is None for n in needs] == [True, False, True] and [s is None for s in states] == [False, True, False]
    eng = Engine(model, max_tokens=256, decode_splits=2)
    assert set(eng.cache.state) == {0, 2} and len(eng.cache.groups) == 1
    w = P.read_safetensors(os.path.join(folder, "model.safetensors"))
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 90, n).tolist() for n in (30, 12)]
    ref = [_toy_plain(w, raw, s) for s in seqs]
    for round_ in range(2):                                       # the second round reuses slots: state must be zeroed
        slots = [eng.new_sequence() for _ in seqs]
        got = host(eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, (20, 5))], "all"))
        want = np.concatenate([ref[0][:20], ref[1][:5]])
        assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max()), round_
        pos = [20, 5]
        if round_ == 1:           # several tokens onto started sequences: the state carries on, the attention
            got = host(eng.step([(slots[0], seqs[0][20:23]), (slots[1], seqs[1][5:6])], "all"))   # layer reads cache + step
            want = np.concatenate([ref[0][20:23], ref[1][5:6]])
            assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())
            pos = [23, 6]
        for _ in range(6):
            got = host(eng.step([(s, [q[p]]) for s, q, p in zip(slots, seqs, pos)]))
            for r in range(2):
                assert np.abs(got[r] - ref[r][pos[r]]).max() < 1e-4 * max(1.0, np.abs(ref[r]).max())
                pos[r] += 1
        for s in slots:
            eng.release(s)
    eng.cache.audit()


# ---- a second toy architecture: a feed-forward with routing and another position encoding ---------

def _define_toy2():
    from quicknn_b200.config.base import (Architecture, ModelConfig, as_float, as_int, register_architecture)
    from quicknn_b200.kernels import ops
    from quicknn_b200.parts import (FEED_FORWARDS, MIXERS, POSITIONS, EmbeddingSpec, FeedForward, HeadSpec, LayerSpec,
                                    Mixer, ModelSpec, PartSpec, Positions, ScheduleEntry, StateNeed)

    @FEED_FORWARDS.register("toy_routed", replace=True)
    class RoutedFF(FeedForward):
        """E small experts; the router's logits are float32, a token goes to its best expert
        and the expert's output is weighted with the softmax probability of that choice."""

        def __init__(self, spec):
            super().__init__(spec)
            p = spec.params
            self.H, self.E, self.I = int(p["hidden_size"]), int(p["experts"]), int(p["inner"])

        @classmethod
        def param_shapes(cls, spec):
            p = spec.params
            H, E, I = int(p["hidden_size"]), int(p["experts"]), int(p["inner"])
            M = cls.PARAM_ROLE_MATRIX
            return {"router": ((E, H), M), "w_in": ((E * I, H), M), "w_out": ((E * H, I), M)}

        def load(self, tensors, compute_dtype, device):
            self.router = tensors["router"].float().contiguous()
            self.w_in = tensors["w_in"].contiguous().view(self.E, self.I, self.H)
            self.w_out = tensors["w_out"].contiguous().view(self.E, self.H, self.I)

        def weight_bytes(self):
            return sum(t.numel() * t.element_size() for t in (self.router, self.w_in, self.w_out))

        def forward(self, x, step):
            logits = ops.linear(x.float().contiguous(), self.router)            # router in float32
            prob = torch.softmax(logits, dim=-1)
            best = prob.argmax(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.E):                                           # a toy: expert by expert
                rows = (best == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                h = ops.linear(x[rows].contiguous(), self.w_in[e].contiguous())
                h = torch.relu(h.float()).to(x.dtype)
                y = ops.linear(h.contiguous(), self.w_out[e].contiguous())
                out[rows] = (y.float() * prob[rows, e].unsqueeze(1)).to(x.dtype)
            return out

    @POSITIONS.register("toy_sinusoid", replace=True)
    class SinusoidAdd(Positions):
        """Adds sin(position * rate_j) to element j: an absolute encoding, nothing rotated."""

        def __init__(self, spec):
            super().__init__(spec)
            self.size, self.base = int(spec.params["size"]), float(spec.params["base"])
            self.rotary_dim, self.inv_freq = 0, None

        def prepare(self, device):
            j = torch.arange(self.size, dtype=torch.float64)
            self.rates = torch.exp(-math.log(self.base) * j / self.size).float().to(device)

        def apply(self, x, tok_pos):
            return (x.float() + torch.sin(tok_pos.float().unsqueeze(1) * self.rates.unsqueeze(0))).to(x.dtype)

        def place(self, qkv, heads, step, line, append=True):
            """What the stock attention mixer calls: the same signal added to every query and key head
            (``size`` = head size), values untouched, then the append."""
            qk = qkv[:, :(heads.n_heads + heads.n_kv_heads) * heads.head_dim].view(qkv.shape[0], -1, heads.head_dim)
            qk.add_(torch.sin(step.tok_pos.float().unsqueeze(1) * self.rates.unsqueeze(0)).unsqueeze(1).to(qkv.dtype))
            if append and line.writes:
                ops.cache_append(qkv, heads.n_heads, heads.n_kv_heads, heads.head_dim, step.tok_pos, step.tok_slot, line)

    @MIXERS.register("toy_posdecay", replace=True)
    class PosDecayMixer(Mixer):
        """The decaying sum of the first toy, over inputs that carry their position."""

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden, self.decay = int(spec.params["hidden_size"]), float(spec.params["decay"])
            pos = spec.params["position"]
            self.position = POSITIONS.get(pos.kind)(pos)

        @classmethod
        def param_shapes(cls, spec):
            h = int(spec.params["hidden_size"])
            return {"mix": ((h, h), cls.PARAM_ROLE_MATRIX)}

        def load(self, tensors, compute_dtype, device):
            self.w = tensors["mix"].contiguous()
            self.position.prepare(device)

        def weight_bytes(self):
            return self.w.numel() * self.w.element_size()

        def state_need(self):
            return StateNeed((self.hidden,), "float32")

        def forward(self, x, step, line):
            xf = self.position.apply(x, step.tok_pos).float()
            out = torch.empty_like(xf)
            for t, s in enumerate(step.tok_slot.cpu().tolist()):
                if s < 0:
                    out[t] = 0
                    continue
                line.state[s].mul_(self.decay).add_(xf[t])
                out[t] = line.state[s]
            return ops.linear(out.to(x.dtype).contiguous(), self.w)

    def _f(conv, **kw):
        return dataclasses.field(default=kw.get("default"), metadata={"convert": conv, "required": "default" not in kw})

    @dataclasses.dataclass(frozen=True)
    class Toy2Config(ModelConfig):
        hidden_size: int = _f(as_int)
        vocab_size: int = _f(as_int)
        n_heads: int = _f(as_int)
        n_kv_heads: int = _f(as_int)
        head_dim: int = _f(as_int)
        rotary_dim: int = _f(as_int)
        inner: int = _f(as_int)
        experts: int = _f(as_int)
        expert_inner: int = _f(as_int)
        decay: float = _f(as_float)
        eps: float = _f(as_float)
        max_position_embeddings: int = _f(as_int)

    def toy2_spec(c):
        H = c.hidden_size
        norm = PartSpec("rmsnorm", {"size": H, "eps": c.eps, "unit_offset": True})
        dense = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": c.inner, "activation": "gelu_tanh"})
        routed = PartSpec("toy_routed", {"hidden_size": H, "experts": c.experts, "inner": c.expert_inner})
        attn = PartSpec("attention", {"hidden_size": H, "n_heads": c.n_heads, "n_kv_heads": c.n_kv_heads,
                                      "head_dim": c.head_dim, "scale": c.head_dim ** -0.5, "softcap": 20.0, "window": 6,
                                      "position": PartSpec("rotary", {"head_dim": c.head_dim, "theta": 500.0,
                                                                      "rotary_dim": c.rotary_dim})})
        posmix = PartSpec("toy_posdecay", {"hidden_size": H, "decay": c.decay,
                                           "position": PartSpec("toy_sinusoid", {"size": H, "base": 50.0})})
        # the stock attention mixer with a position part that is not a rotation: nothing of the mixer changes
        attn_abs = PartSpec("attention", {"hidden_size": H, "n_heads": c.n_heads, "n_kv_heads": c.n_kv_heads,
                                          "head_dim": c.head_dim, "scale": c.head_dim ** -0.5, "softcap": None,
                                          "window": None,
                                          "position": PartSpec("toy_sinusoid", {"size": c.head_dim, "base": 30.0})})
        n4 = {k: norm for k in ("pre_mixer", "pre_ff")}
        l0 = {"mixer.mix": "a.mix", "ff.router": "a.router", "ff.w_in": "a.w_in", "ff.w_out": "a.w_out",
              "norms.pre_mixer.weight": "a.n1", "norms.pre_ff.weight": "a.n2"}
        l1 = {f"mixer.{x}_proj": f"b.{x}" for x in "qkvo"}
        l1.update({f"ff.{n}_proj": f"b.{n}" for n in ("gate", "up", "down")})
        l1.update({"norms.pre_mixer.weight": "b.n1", "norms.pre_ff.weight": "b.n2"})
        l2 = {k.replace("b.", "c."): v.replace("b.", "c.") for k, v in l1.items()}
        layers = (LayerSpec(PartSpec("prenorm", {}), posmix, routed, n4, l0),
                  LayerSpec(PartSpec("prenorm", {}), attn, dense, n4, l1),
                  LayerSpec(PartSpec("prenorm", {}), attn_abs, dense, n4, l2))
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 2))
        return ModelSpec("Toy2ForTest", H, EmbeddingSpec(c.vocab_size, H, 1.0, "emb"), layers, schedule,
                         HeadSpec(c.vocab_size, H, True, None, None, norm, "nf"), c.max_position_embeddings,
                         init_std=0.3, init_norm_std=0.2)

    arch = register_architecture(Architecture("Toy2ForTest", Toy2Config, toy2_spec), replace=True)
    return arch, Toy2Config


def _toy2_plain(w, cfg, ids):
    """The second toy model in NumPy, whole sequence."""
    H, nh, nkv, hd, rd = cfg["hidden_size"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["rotary_dim"]
    E, EI = cfg["experts"], cfg["expert_inner"]
    norm = lambda x, g: x / np.sqrt((x * x).mean(-1, keepdims=True) + cfg["eps"]) * (1.0 + g)  # noqa: E731
    x = w["emb"][ids].astype(np.float64)
    T = len(ids)
    pos = np.arange(T)
    # layer 0: positions added, decaying sum, then the routed feed-forward
    n = norm(x, w["a.n1"])
    rates = np.exp(-math.log(50.0) * np.arange(H) / H).astype(np.float32).astype(np.float64)
    n = n + np.sin(pos[:, None] * rates[None, :])
    s, out = np.zeros(H), np.zeros_like(n)
    for t in range(T):
        s = cfg["decay"] * s + n[t]
        out[t] = s
    x = x + out @ w["a.mix"].T
    n = norm(x, w["a.n2"])
    logits = n @ w["a.router"].T
    prob = np.exp(logits - logits.max(-1, keepdims=True))
    prob /= prob.sum(-1, keepdims=True)
    best = prob.argmax(-1)
    w_in, w_out = w["a.w_in"].reshape(E, EI, H), w["a.w_out"].reshape(E, H, EI)
    y = np.zeros_like(x)
    for t in range(T):
        e = best[t]
        y[t] = (w_out[e] @ np.maximum(w_in[e] @ n[t], 0.0)) * prob[t, e]
    x = x + y
    # layer 1: windowed, softcapped attention with a partly rotated head, dense feed-forward
    n = norm(x, w["b.n1"])
    q = (n @ w["b.q"].T).reshape(T, nh, hd)
    k = (n @ w["b.k"].T).reshape(T, nkv, hd)
    v = (n @ w["b.v"].T).reshape(T, nkv, hd)
    rot = lambda z: np.concatenate([P.rope(z[..., :rd], pos, 500.0), z[..., rd:]], axis=-1)  # noqa: E731
    a = P.attention(rot(q), rot(k), v, hd ** -0.5, 20.0, 6).reshape(T, -1)
    x = x + a @ w["b.o"].T
    n = norm(x, w["b.n2"])
    x = x + (P.gelu_tanh(n @ w["b.gate"].T) * (n @ w["b.up"].T)) @ w["b.down"].T
    # layer 2: full attention whose queries and keys carry an added position signal, dense feed-forward
    n = norm(x, w["c.n1"])
    sig = np.sin(pos[:, None] * np.exp(-math.log(30.0) * np.arange(hd) / hd).astype(np.float32).astype(np.float64)[None, :])
    q = (n @ w["c.q"].T).reshape(T, nh, hd) + sig[:, None, :]
    k = (n @ w["c.k"].T).reshape(T, nkv, hd) + sig[:, None, :]
    v = (n @ w["c.v"].T).reshape(T, nkv, hd)
    x = x + P.attention(q, k, v, hd ** -0.5, None, None).reshape(T, -1) @ w["c.o"].T
    n = norm(x, w["c.n2"])
    x = x + (P.gelu_tanh(n @ w["c.gate"].T) * (n @ w["c.up"].T)) @ w["c.down"].T
    return norm(x, w["nf"]) @ w["emb"].T, best


def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    """A feed-forward with a router and experts, a position part that is not a rotation, and an
    attention layer with a partly rotated head, a window and a softcap: chosen layer by layer through
    the registries, defined in this file, stepped by the unchanged engine."""
    from quicknn_b200.engine import Engine, Model
    from quicknn_b200.weights import write_model_folder
    arch, Toy2Config = _define_toy2()
    raw = dict(architectures=["Toy2ForTest"], hidden_size=48, vocab_size=70, n_heads=4, n_kv_heads=2, head_dim=16,
               rotary_dim=8, inner=72, experts=3, expert_inner=40, decay=0.6, eps=1e-5, max_position_embeddings=128)
    cfg = Toy2Config.from_dict(raw)
    folder = write_model_folder(str(tmp_path / "toy2"), arch, cfg, 11, torch.float32)
    model = Model.from_folder(folder, "float32", DEV)
    eng = Engine(model, max_tokens=256, decode_splits=2)
    w = P.read_safetensors(os.path.join(folder, "model.safetensors"))
    rng = np.random.default_rng(3)
    seqs = [rng.integers(0, 70, n).tolist() for n in (26, 9, 17)]
    refs = [_toy2_plain(w, raw, s) for s in seqs]
    assert len(set(np.concatenate([b for _, b in refs]).tolist())) > 1          # the router does choose
    slots = [eng.new_sequence() for _ in seqs]
    first = (15, 4, 17)
    got = host(eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, first)], "all"))
    want = np.concatenate([r[:n] for (r, _), n in zip(refs, first)])
    assert np.abs(got - want).max() < 2e-4 * max(1.0, np.abs(want).max())
    eng.release(slots[2])                                                        # the whole one is done
    pos = [15, 4]
    for _ in range(5):
        got = host(eng.step([(s, [q[p]]) for s, q, p in zip(slots[:2], seqs[:2], pos)]))
        for r in range(2):
            assert np.abs(got[r] - refs[r][0][pos[r]]).max() < 2e-4 * max(1.0, np.abs(refs[r][0]).max())
            pos[r] += 1
    for s in slots[:2]:
        eng.release(s)
    eng.cache.audit()
