"""One layer at the layer sizes of Gemma 2 2B, 9B and 27B (hidden, heads, head size, feed-forward
width, window, scale factors as in those models; one layer and a small vocabulary to keep the files
small), random weights, against the plain implementation: a whole prompt longer than a 64-row
attention tile, then tokens one by one, in float32 and in bfloat16.  These are the sizes at which
the tensor-core kernels (tcgen05 products, head-size 256 and 128 attention) run in the benchmark."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SIZES = {
    "2b": dict(hidden_size=2304, intermediate_size=9216, num_attention_heads=8, num_key_value_heads=4, head_dim=256,
               query_pre_attn_scalar=256),
    "9b": dict(hidden_size=3584, intermediate_size=14336, num_attention_heads=16, num_key_value_heads=8, head_dim=256,
               query_pre_attn_scalar=256),
    "27b": dict(hidden_size=4608, intermediate_size=36864, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
                query_pre_attn_scalar=144),
}


def _folder(tmp, name, storage):
    from quicknn_b200.config import GEMMA2, Gemma2Config
    from quicknn_b200.weights import write_model_folder
    raw = dict(architectures=["Gemma2ForCausalLM"], model_type="gemma2", vocab_size=2048, num_hidden_layers=1,
               max_position_embeddings=8192, rope_theta=10000.0, rms_norm_eps=1e-6, sliding_window=64,
               attn_logit_softcapping=50.0, final_logit_softcapping=30.0, eos_token_id=1, initializer_range=0.02,
               **SIZES[name])
    cfg = Gemma2Config.from_dict(raw)
    d = os.path.join(str(tmp), f"{name}_{storage}")
    write_model_folder(d, GEMMA2, cfg, seed={"2b": 2, "9b": 3, "27b": 4}[name],
                       dtype=torch.float32 if storage == "float32" else torch.bfloat16, norm_std=0.1)
    return d


@pytest.mark.parametrize("name", ["2b", "9b", "27b"])
def test_one_layer_at_model_sizes(tmp_path, name):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from plain.gemma2_plain import PlainGemma2
    from quicknn_b200.engine import Engine, Model
    folder = _folder(tmp_path, name, "bfloat16")          # bf16 weights; float32 mode widens them exactly
    plain = PlainGemma2(folder)
    rng = np.random.default_rng(7)
    seqs = [rng.integers(1, 2048, n).tolist() for n in (150, 37)]
    ref = [plain.logits(s) for s in seqs]
    for dtype in ("float32", "bfloat16"):
        eng = Engine(Model.from_folder(folder, dtype, DEV), max_tokens=512)
        slots = [eng.new_sequence() for _ in seqs]
        cut = [142, 30]
        got = eng.step([(s, q[:c]) for s, q, c in zip(slots, seqs, cut)], "all").cpu().numpy()
        want = np.concatenate([r[:c] for r, c in zip(ref, cut)])
        ok, err, tol = close(got, want, dtype)
        assert ok, (name, dtype, "prompt", err, tol)
        pos = list(cut)
        for _ in range(7):
            toks = torch.tensor([q[p] for q, p in zip(seqs, pos)], dtype=torch.int32, device=DEV)
            got = eng.decode(slots, toks).cpu().numpy()
            for r in range(2):
                ok, err, tol = close(got[r], ref[r][pos[r]], dtype)
                assert ok, (name, dtype, "decode", r, pos[r], err, tol)
                pos[r] += 1
        del eng
        torch.cuda.empty_cache()
