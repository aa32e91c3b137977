"""Shared by the tests: tiny configurations, model folders in temporary places, traces."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from binfer_b200.config import Qwen3Config
from binfer_b200.weights import TensorSource, write_model_dir

# Two tiny configurations that differ in every size and option, and a third with a window.
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
    num_attention_heads=4, num_key_value_heads=2, intermediate_size=128, vocab_size=256,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False,
    max_position_embeddings=512, hidden_act="silu", attention_bias=False)          # head_dim = 64/4
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
    num_attention_heads=6, num_key_value_heads=1, head_dim=32, intermediate_size=160,
    vocab_size=300, rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=1024, hidden_act="silu",
    attention_bias=False)
TINY_W = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=80,
    num_attention_heads=5, num_key_value_heads=5, head_dim=48, intermediate_size=112,
    vocab_size=270, rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
    use_sliding_window=True, sliding_window=24,
    layer_types=["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
    max_position_embeddings=2048, hidden_act="silu", attention_bias=False)

# head size 128 and pages of 16: the sizes the TMA / tcgen05 kernels are written for
TINY_M = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=256,
    num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=512,
    vocab_size=500, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=4096, hidden_act="silu",
    attention_bias=False)

# the same sizes with a window on two of three layers: the TMA / tcgen05 attention kernels
# with keys that fall out of the window, and pages that are given back while a request runs
TINY_V = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=256,
    num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=384,
    vocab_size=410, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True,
    use_sliding_window=True, sliding_window=150,
    layer_types=["sliding_attention", "full_attention", "sliding_attention"],
    max_position_embeddings=4096, hidden_act="silu", attention_bias=False)

# sizes that are no power of two at the scale where the decode step's cluster products, the
# persistent decode attention and the tcgen05 head product run: a width of 1536, 4480 inner
# features, a vocabulary of 5001.  (One layer: at this width two layers' bfloat16 rounding
# alone, with every product on the library, is 1.05e-2 of the logits' rms, over the bound
# that the other configurations are held to.)
TINY_O = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=1, hidden_size=1536,
    num_attention_heads=16, num_key_value_heads=2, head_dim=128, intermediate_size=4480,
    vocab_size=5001, rope_theta=5e5, rms_norm_eps=2e-6, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=4096, hidden_act="silu",
    attention_bias=False)

# wide enough (2048 inputs to the output and down projections) for the decode step's
# split-K cluster products, and with them the products that prepare the next norm
TINY_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=1024,
    num_attention_heads=16, num_key_value_heads=4, head_dim=128, intermediate_size=2048,
    vocab_size=600, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=4096, hidden_act="silu",
    attention_bias=False)

# the layer sizes of the Qwen3-8B shape (hidden 4096, 32/8 heads of 128, 12288 inner
# features, an untied head over 151936 words) with fewer layers: two.  What a decode or a
# prefill step of the full model launches, kernel for kernel, but small enough to compare
# with the plain implementation.
QWEN3_8B_TWO_LAYERS = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
    vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=40960, hidden_act="silu",
    attention_bias=False)

# the layer sizes of the Qwen3-1.7B shape (tied head), two layers of its 28
QWEN3_1P7B_TWO_LAYERS = dict(
    QWEN3_8B_TWO_LAYERS, hidden_size=2048, num_attention_heads=16, num_key_value_heads=8,
    intermediate_size=6144, tie_word_embeddings=True)

# for the smoke test: small, but of the sizes that a decode step's tcgen05 kernels take
# (2048 inputs to every projection, heads of 128, a head product over more than 65536 words)
SMOKE_WIDE = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=2048,
    num_attention_heads=16, num_key_value_heads=4, head_dim=128, intermediate_size=3072,
    vocab_size=66001, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True,
    use_sliding_window=False, max_position_embeddings=4096, hidden_act="silu",
    attention_bias=False)

TINY = {
    "S": dict(raw=SMOKE_WIDE, std=0.02, norm_std=0.05, page_size=64, seed=88),
    "O": dict(raw=TINY_O, std=0.03, norm_std=0.05, page_size=64, seed=77),
    "V": dict(raw=TINY_V, std=0.05, norm_std=0.02, page_size=32, seed=66),
    "F": dict(raw=TINY_F, std=0.03, norm_std=0.05, page_size=64, seed=55),
    "M": dict(raw=TINY_M, std=0.05, norm_std=0.02, page_size=16, seed=44),
    "A": dict(raw=TINY_A, std=0.02, norm_std=0.01, page_size=16, seed=11),
    "B": dict(raw=TINY_B, std=0.05, norm_std=0.05, page_size=8, seed=22),
    "W": dict(raw=TINY_W, std=0.04, norm_std=0.03, page_size=4, seed=33),
}


def make_model_dir(tmp_path, which: str, dtype=torch.float32) -> str:
    t = TINY[which]
    cfg = Qwen3Config.from_dict(t["raw"])
    d = os.path.join(str(tmp_path), f"tiny_{which}_{str(dtype).split('.')[-1]}")
    write_model_dir(cfg, d, seed=t["seed"], std=t["std"], norm_std=t["norm_std"], dtype=dtype)
    return d


def read_model_dir(d: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    with open(os.path.join(d, "config.json")) as f:
        raw = json.load(f)
    src = TensorSource.from_dir(d)
    w = {n: src.get(n).clone() for n in src.shapes}
    src.close()
    return raw, w


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest absolute difference over the largest reference magnitude."""
    return float((got.double() - ref.double()).abs().max() / ref.double().abs().max())


def rel_rms(got: torch.Tensor, ref: torch.Tensor) -> float:
    d = (got.double() - ref.double())
    return float(d.pow(2).mean().sqrt() / ref.double().pow(2).mean().sqrt())


def assert_greedy_within_rounding(raw, w, prompts, outs, bound=3e-2):
    """Every generated token is the plain implementation's choice at its place, given the
    tokens before it, or, where the plain logits of the best tokens lie closer together than
    bfloat16 rounding can tell apart (``bound`` of the largest logit), one of those."""
    import qwen3_plain as P
    for p, out in zip(prompts, outs):
        logits = P.forward(raw, w, list(p) + list(out), dtype=torch.float64)
        for n, tok in enumerate(out):
            row = logits[len(p) - 1 + n]
            slack = bound * float(row.abs().max())
            assert float(row[tok]) >= float(row.max()) - slack, (
                f"token {n} of a prompt of {len(p)}: {tok} has plain logit {float(row[tok]):.4f}, "
                f"the best ({int(row.argmax())}) {float(row.max()):.4f}")


# ------------------------------------------------------------------------ traces
def trace_whole(reqs: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, logits wanted everywhere."""
    steps = []
    for i, (rid, toks) in enumerate(reqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks,
                                              "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def trace_decode_tail(reqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps, s = [], 0
    for rid, toks in reqs.items():
        n = max(1, len(toks) - tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:n],
                                              "want": list(range(n))}], "end": []})
        s += 1
        for i in range(n, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            s += 1
        if n == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(reqs: Dict[str, List[int]], sizes: Sequence[int] = (7, 5, 3, 2, 11, 2, 16, 9)
                   ) -> List[dict]:
    """Portions of changing size, down to two tokens."""
    steps, s, k = [], 0, 0
    for rid, toks in reqs.items():
        a = 0
        while a < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - a)
            k += 1
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[a:a + n],
                                                  "want": list(range(n))}],
                          "end": [rid] if a + n == len(toks) else []})
            a += n
            s += 1
    return steps


def trace_mixed(reqs: Dict[str, List[int]], max_live: int = 4, tail: int = 10,
                sizes: Sequence[int] = (7, 2, 13, 5, 3, 9), skip_every: int = 5) -> List[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside decoded tokens of
    others; a request sits out a step now and then; finished ones make room for new ones."""
    waiting = list(reqs.items())
    live: List[List] = []          # [rid, tokens, done]
    steps, s, k = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live.append([rid, toks, 0])
            if len(live) < max_live and s % 2 == 0:
                break               # stagger arrivals
        entries, end = [], []
        for j, r in enumerate(live):
            rid, toks, done = r
            if (s + j) % skip_every == skip_every - 1 and len(live) > 1:
                continue            # this request sits the step out
            left = len(toks) - done
            n = 1 if left <= tail else min(sizes[k % len(sizes)], left - tail)
            k += 1
            entries.append({"id": rid, "tokens": toks[done:done + n], "want": list(range(n))})
            r[2] = done + n
            if r[2] == len(toks):
                end.append(rid)
        if entries:
            steps.append({"step": s, "entries": entries, "end": end})
        live = [r for r in live if r[2] < len(r[1])]
        s += 1
    return steps


def thin_wants(steps: List[dict], keep) -> List[dict]:
    """The same steps with logits wanted only where ``keep(request, position)`` says so."""
    pos: Dict[str, int] = {}
    out = []
    for st in steps:
        entries = []
        for e in st["entries"]:
            a = pos.get(e["id"], 0)
            entries.append(dict(e, want=[w for w in e["want"] if keep(e["id"], a + w)]))
            pos[e["id"]] = a + len(e["tokens"])
        for rid in st["end"]:
            pos.pop(rid, None)
        out.append(dict(st, entries=entries))
    return out


def peak_pages(steps: List[dict], page_size: int) -> int:
    """Most pages held at once by a full-attention cache group while replaying ``steps``."""
    held: Dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // page_size) for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def run_trace(runner, steps: List[dict]) -> Dict[Tuple[str, int], torch.Tensor]:
    """Replay ``steps`` on a ModelRunner; logits by (request, position), on the CPU."""
    from binfer_b200.engine.runner import StepItem
    pos: Dict[str, int] = {}
    out: Dict[Tuple[str, int], torch.Tensor] = {}
    for st in steps:
        items = []
        for e in st["entries"]:
            if e["id"] not in pos:
                runner.add_request(e["id"])
                pos[e["id"]] = 0
            items.append(StepItem(e["id"], e["tokens"], e["want"]))
        logits = runner.step(items).float().cpu()
        runner.check_errors()
        r = 0
        for e in st["entries"]:
            for w in e["want"]:
                out[(e["id"], pos[e["id"]] + w)] = logits[r]
                r += 1
            pos[e["id"]] += len(e["tokens"])
        for rid in st["end"]:
            runner.free_request(rid)
            del pos[rid]
        runner.cache.check_consistent()
    return out


# ------------------------------------------------------------------ the hybrid design
def _guk_attn(heads, kv_heads, dim, vdim, window, pool, rot_dims, base=10000.0, scale=None,
              kv_from=None, layout=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "mask": {"size": window, "pool": pool},
         "rot": {"base": base, "dims": rot_dims},
         "scale": dim ** -0.5 if scale is None else scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    if layout is not None:
        m["rot"]["layout"] = layout
    return m


def _guk_layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _guk_mlstm(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


# memory / attention alternating; a memory layer with a feed-forward, an attention layer
# without; the second attention layer reads the first one's keys and values
GUK_A = {"architecture": "Gukidra", "vocab": 300, "width": 64, "norm": {"eps": 1e-6},
         "embedding": {"scale": 6.0},
         "layers": [_guk_layer("mlstm", _guk_mlstm(2, 16, 32, 8.0)),
                    _guk_layer("attention", _guk_attn(4, 2, 32, 16, 24, 4, 16), ff=96),
                    _guk_layer("mlstm", _guk_mlstm(2, 16, 32, 8.0), ff=80),
                    _guk_layer("attention", _guk_attn(4, 2, 32, 16, 24, 4, 16, kv_from=1))]}
# attention first; no grouping; values larger than keys and no multiple of 32; a window
# smaller than the pooled block; the reader has a mask of its own (wider window, other block);
# one memory head; no embedding scale
GUK_B = {"architecture": "Gukidra", "vocab": 211, "width": 48, "norm": {"eps": 1e-5},
         "embedding": {"scale": 1.0},
         "layers": [_guk_layer("attention", _guk_attn(3, 3, 24, 40, 7, 8, 24, base=500.0, scale=0.3),
                               ff=64),
                    _guk_layer("mlstm", _guk_mlstm(1, 40, 24, 5.0)),
                    _guk_layer("attention", _guk_attn(3, 3, 24, 40, 20, 5, 24, base=500.0,
                                                      scale=0.25, kv_from=0), ff=72),
                    _guk_layer("mlstm", _guk_mlstm(3, 8, 8, 15.0), ff=56)]}
# a window of one token and blocks of one token: every earlier token is seen as a block;
# one key/value head; interleaved pairs
GUK_C = {"architecture": "Gukidra", "vocab": 150, "width": 32, "norm": {"eps": 1e-6},
         "embedding": {"scale": 3.0},
         "layers": [_guk_layer("attention", _guk_attn(2, 1, 16, 16, 1, 1, 8, layout="interleaved"),
                               ff=48),
                    _guk_layer("mlstm", _guk_mlstm(2, 8, 16, 10.0)),
                    _guk_layer("attention", _guk_attn(2, 1, 16, 16, 5, 3, 16), ff=40)]}
# wider, for bfloat16: heads of 64 and 128, a window of 64 with blocks of 16
GUK_D = {"architecture": "Gukidra", "vocab": 500, "width": 256, "norm": {"eps": 1e-6},
         "embedding": {"scale": 10.0},
         "layers": [_guk_layer("mlstm", _guk_mlstm(4, 64, 64, 12.0)),
                    _guk_layer("attention", _guk_attn(4, 1, 64, 128, 64, 16, 32), ff=512),
                    _guk_layer("mlstm", _guk_mlstm(2, 32, 128, 12.0)),
                    _guk_layer("attention", _guk_attn(4, 1, 64, 128, 64, 16, 32, kv_from=1),
                               ff=384)]}

# sizes that are multiples of two only: a width of 50, heads of 10 and 6, a vocabulary of 131
GUK_E = {"architecture": "Gukidra", "vocab": 131, "width": 50, "norm": {"eps": 1e-6},
         "embedding": {"scale": 2.5},
         "layers": [_guk_layer("mlstm", _guk_mlstm(2, 6, 10, 7.0), ff=34),
                    _guk_layer("attention", _guk_attn(2, 1, 10, 6, 9, 2, 6, base=3000.0), ff=46),
                    _guk_layer("attention", _guk_attn(2, 1, 10, 6, 13, 3, 6, base=3000.0,
                                                      kv_from=1))]}

GUK = {
    "E": dict(raw=GUK_E, std=0.12, norm_std=0.1, page_size=16, seed=9),
    "A": dict(raw=GUK_A, std=0.08, norm_std=0.1, page_size=16, seed=5),
    "B": dict(raw=GUK_B, std=0.1, norm_std=0.1, page_size=4, seed=6),
    "C": dict(raw=GUK_C, std=0.12, norm_std=0.1, page_size=8, seed=7),
    "D": dict(raw=GUK_D, std=0.05, norm_std=0.05, page_size=16, seed=8),
}


def make_gukidra_dir(tmp_path, which, dtype=torch.float32, raw=None, tweak=None, tag="") -> str:
    """A folder with config.json and random weights of a hybrid configuration; ``tweak(w)``
    may change the tensors (a name -> tensor dictionary) before they are written."""
    from binfer_b200.config import GukidraConfig
    from binfer_b200.parts.model import param_specs_for
    from binfer_b200.weights import random_tensors, save_file
    t = GUK[which]
    raw = raw or t["raw"]
    cfg = GukidraConfig.from_dict(raw)
    d = os.path.join(str(tmp_path), f"guk_{which}{tag}_{str(dtype).split('.')[-1]}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    w = random_tensors(param_specs_for(cfg.to_spec()), t["seed"], t["std"], t["norm_std"], dtype)
    if tweak is not None:
        tweak(w)
    save_file(w, os.path.join(d, "model.safetensors"))
    return d


# ------------------------------------------------------------ the side-by-side design
def _fik_left(heads, kv_heads, dim, vdim, window, keep, rot_dims, conv=3, base=10000.0,
              scale=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
         "mask": {"size": window, "keep_first": keep},
         "rot": {"base": base, "dims": rot_dims},
         "scale": dim ** -0.5 if scale is None else scale}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def _fik_right(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
            "rot": {"base": base, "dims": rot_dims}}


def _fik_moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _fik_layer(left, right, mlp=None, ls=1.0, rs=1.0):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}}


# grouped heads, values smaller than keys, a window of 24 that keeps 5 tokens, three taps;
# one layer without a feed-forward
FIK_A = {"architecture": "Fikotar", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
         "logit_scale": 0.5,
         "layers": [_fik_layer(_fik_left(4, 2, 32, 16, 24, 5, 16, scaling=(8.0, 1.0, 4.0, 64)),
                               _fik_right(2, 16, 32, (0.9, 0.99), 16), _fik_moe(4, 2, 48, 64),
                               ls=0.7, rs=1.2),
                    _fik_layer(_fik_left(4, 2, 32, 16, 24, 5, 16, scaling=(8.0, 1.0, 4.0, 64)),
                               _fik_right(2, 16, 32, (0.95, 0.999), 16), None, ls=1.1, rs=0.6),
                    _fik_layer(_fik_left(2, 1, 16, 48, 9, 0, 8, conv=2),
                               _fik_right(1, 40, 24, (0.97,), 20), _fik_moe(5, 1, 40))]}
# no grouping; values larger than keys and no multiple of 32; a window smaller than a page
# and more kept tokens than a page holds; four taps; every expert chosen; a decay of one;
# the whole head rotated; no logit scale
FIK_B = {"architecture": "Fikotar", "vocab": 211, "width": 48, "norm": {"eps": 1e-6},
         "layers": [_fik_layer(_fik_left(3, 3, 24, 40, 3, 6, 24, conv=4, base=500.0, scale=0.3),
                               _fik_right(3, 8, 8, (1.0, 0.5, 0.98), 8, base=500.0),
                               _fik_moe(3, 3, 56, 24)),
                    _fik_layer(_fik_left(3, 1, 24, 40, 20, 1, 12, conv=0, base=500.0, scale=0.25,
                                         scaling=(2.0, 0.5, 3.0, 40)),
                               _fik_right(2, 12, 20, (0.93, 0.9995), 4, base=500.0),
                               _fik_moe(6, 2, 32, 72), ls=0.5, rs=0.5)]}
# sizes that are multiples of two only: a width of 50, heads of 10 and 6, a vocabulary of 131;
# a window of one token; a convolution of one tap (a factor per channel)
FIK_C = {"architecture": "Fikotar", "vocab": 131, "width": 50, "norm": {"eps": 1e-5},
         "logit_scale": 2.0,
         "layers": [_fik_layer(_fik_left(2, 1, 10, 6, 1, 2, 6, conv=2, base=3000.0),
                               _fik_right(2, 6, 10, (0.9, 0.8), 6, base=3000.0),
                               _fik_moe(2, 1, 34, 46), ls=1.0, rs=1.0),
                    _fik_layer(_fik_left(5, 5, 10, 10, 13, 0, 10, conv=1, base=3000.0),
                               _fik_right(1, 10, 6, (0.99,), 2, base=3000.0), None)]}
# wider, for bfloat16: heads of 64 and 128, a window of 64 that keeps four tokens
FIK_D = {"architecture": "Fikotar", "vocab": 500, "width": 256, "norm": {"eps": 1e-5},
         "logit_scale": 0.3,
         "layers": [_fik_layer(_fik_left(4, 1, 64, 128, 64, 4, 32, scaling=(4.0, 1.0, 4.0, 256)),
                               _fik_right(4, 64, 64, (0.97, 0.99, 0.995, 0.999), 64),
                               _fik_moe(8, 2, 128, 256), ls=0.8, rs=0.9),
                    _fik_layer(_fik_left(8, 4, 32, 32, 40, 0, 32, conv=2),
                               _fik_right(2, 32, 128, (0.98, 0.9999), 16),
                               _fik_moe(4, 3, 192), ls=1.0, rs=0.5)]}

FIK = {
    "A": dict(raw=FIK_A, std=0.08, norm_std=0.1, page_size=16, seed=15),
    "B": dict(raw=FIK_B, std=0.1, norm_std=0.1, page_size=4, seed=16),
    "C": dict(raw=FIK_C, std=0.12, norm_std=0.1, page_size=8, seed=17),
    "D": dict(raw=FIK_D, std=0.05, norm_std=0.05, page_size=16, seed=18),
}


def make_fikotar_dir(tmp_path, which, dtype=torch.float32, raw=None, tweak=None, tag="") -> str:
    """A folder with config.json and random weights of a side-by-side configuration;
    ``tweak(w)`` may change the tensors (a name -> tensor dictionary) before they are written."""
    from binfer_b200.config import FikotarConfig
    from binfer_b200.parts.model import param_specs_for
    from binfer_b200.weights import random_tensors, save_file
    t = FIK[which]
    raw = raw or t["raw"]
    cfg = FikotarConfig.from_dict(raw)
    d = os.path.join(str(tmp_path), f"fik_{which}{tag}_{str(dtype).split('.')[-1]}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    w = random_tensors(param_specs_for(cfg.to_spec()), t["seed"], t["std"], t["norm_std"], dtype)
    if tweak is not None:
        tweak(w)
    save_file(w, os.path.join(d, "model.safetensors"))
    return d


# ----------------------------------------------------------------- the looped design
def _ket_latent(heads, dim, rot_dim, vdim, rank, base=10000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
            "rot": {"base": base, "dims": rot_dim},
            "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}


def _ket_delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _ket_left(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, scale=None, softcap=None,
              scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "rot": {"base": base, "dims": rot_dims},
         "scale": dim ** -0.5 if scale is None else scale}
    if softcap is not None:
        m["softcap"] = softcap
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def _ket_right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _ket_layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _ket_parallel(left, right, ls=1.0, rs=1.0, ff=None):
    return _ket_layer("parallel", {"left": left, "right": right, "left_scale": ls,
                                   "right_scale": rs}, ff)


# the delta rule first; the first two layers walked twice; grouped heads; stretched waves and a
# soft cap; the last layer without a feed-forward
KET_A = {"architecture": "Ketopel", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
         "embedding": {"scale": 2.0}, "loop": {"start": 0, "stop": 2, "times": 2},
         "layers": [_ket_layer("delta", _ket_delta(4, 2, 16, 24, 3), ff=96),
                    _ket_parallel(_ket_left(4, 2, 32, 16, 16, scale=0.2, softcap=20.0,
                                            scaling=(8.0, 64, 4.0, 1.0)),
                                  _ket_right(2, 16, 32, (0.9, 0.99)), ls=0.7, rs=1.2, ff=80),
                    _ket_layer("latent_attention", _ket_latent(3, 24, 8, 20, 40, scale=0.2))]}
# the loop runs to the last layer, three times; no grouping anywhere; values larger than keys
# and no multiple of 32; the whole head rotated, no stretching, no soft cap; a decay of one;
# convolutions of four taps and of one; a layer without a feed-forward inside the loop
KET_B = {"architecture": "Ketopel", "vocab": 211, "width": 48, "norm": {"eps": 1e-6},
         "embedding": {"scale": 1.0}, "loop": {"start": 1, "stop": 4, "times": 3},
         "layers": [_ket_layer("latent_attention", _ket_latent(2, 16, 16, 16, 24, base=500.0), ff=64),
                    _ket_parallel(_ket_left(3, 3, 24, 40, 24, base=500.0, scale=0.3),
                                  _ket_right(3, 8, 8, (1.0, 0.5, 0.98)), ls=0.5, rs=0.5),
                    _ket_layer("delta", _ket_delta(3, 3, 8, 8, 4), ff=56),
                    _ket_layer("delta", _ket_delta(2, 1, 40, 12, 1), ff=40)]}
# sizes that are multiples of two only: a width of 50, heads of 10 and 6, a vocabulary of 131;
# one head; a "loop" of one pass over the last layer; no embedding scale given
KET_C = {"architecture": "Ketopel", "vocab": 131, "width": 50, "norm": {"eps": 1e-5},
         "loop": {"start": 2, "stop": 3, "times": 1},
         "layers": [_ket_layer("delta", _ket_delta(2, 1, 6, 10, 2), ff=34),
                    _ket_layer("latent_attention", _ket_latent(1, 10, 6, 6, 14, base=3000.0), ff=46),
                    _ket_parallel(_ket_left(2, 1, 10, 6, 6, base=3000.0, softcap=5.0),
                                  _ket_right(1, 10, 6, (0.95,)), ff=38)]}
# wider, for bfloat16: a latent of 192 with 32 rotated sizes, delta-rule keys of 128 and of 160;
# the loop walks the two delta rule layers at the end
KET_D = {"architecture": "Ketopel", "vocab": 500, "width": 192, "norm": {"eps": 1e-5},
         "embedding": {"scale": 4.0}, "loop": {"start": 2, "stop": 4, "times": 2},
         "layers": [_ket_layer("latent_attention", _ket_latent(4, 64, 32, 64, 192), ff=512),
                    _ket_parallel(_ket_left(8, 4, 64, 64, 32, scale=0.11, softcap=50.0,
                                            scaling=(4.0, 256, 16.0, 1.0)),
                                  _ket_right(4, 64, 32, (0.97, 0.99, 0.995, 0.999)), ls=0.8,
                                  rs=0.9, ff=320),
                    _ket_layer("delta", _ket_delta(4, 2, 128, 64, 4), ff=384),
                    _ket_layer("delta", _ket_delta(2, 2, 160, 48, 2), ff=256)]}

KET = {
    "A": dict(raw=KET_A, std=0.08, norm_std=0.1, page_size=16, seed=25),
    "B": dict(raw=KET_B, std=0.1, norm_std=0.1, page_size=4, seed=26),
    "C": dict(raw=KET_C, std=0.12, norm_std=0.1, page_size=8, seed=27),
    "D": dict(raw=KET_D, std=0.05, norm_std=0.05, page_size=16, seed=28),
}


def make_ketopel_dir(tmp_path, which, dtype=torch.float32, raw=None, tweak=None, tag="") -> str:
    """A folder with config.json and random weights of a looped configuration; ``tweak(w)``
    may change the tensors (a name -> tensor dictionary) before they are written."""
    from binfer_b200.config import KetopelConfig
    from binfer_b200.parts.model import param_specs_for
    from binfer_b200.weights import random_tensors, save_file
    t = KET[which]
    raw = raw or t["raw"]
    cfg = KetopelConfig.from_dict(raw)
    d = os.path.join(str(tmp_path), f"ket_{which}{tag}_{str(dtype).split('.')[-1]}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    w = random_tensors(param_specs_for(cfg.to_spec()), t["seed"], t["std"], t["norm_std"], dtype)
    if tweak is not None:
        tweak(w)
    save_file(w, os.path.join(d, "model.safetensors"))
    return d


# ------------------------------------------------- the design with a state space layer
def _fol_latent(heads, dim, rot_dim, vdim, rank, q_rank, base=10000.0, scale=None, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
            "q_rank": q_rank, "rot": {"base": base, "dims": rot_dim if dims is None else dims},
            "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}


def _fol_attn(heads, kv_heads, dim, vdim, window, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "mask": {"size": window}, "scale": dim ** -0.5 if scale is None else scale}


def _fol_mamba(heads, groups, state, vdim, conv, norm_groups):
    return {"heads": heads, "groups": groups, "state": state, "vdim": vdim, "conv": conv,
            "norm_groups": norm_groups}


def _fol_moe(experts, top, ff, identity=0, groups=None, scale=1.0, shared=None):
    router = {"experts": experts, "top": top, "identity": identity, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router,
            "shared": None if shared is None else {"ff": shared}}


def _fol_layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# the state space layer first, two heads a group; nine router outputs in three groups, one of
# them an identity expert; a window of 24; the last layer without a feed-forward
FOL_A = {"architecture": "Folivik", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
         "layers": [_fol_layer("mamba2", _fol_mamba(4, 2, 16, 24, 3, 2),
                               _fol_moe(8, 2, 32, identity=1, groups=(3, 2), scale=1.5, shared=48)),
                    _fol_layer("attention", _fol_attn(4, 2, 32, 16, 24, scale=0.3),
                               _fol_moe(6, 3, 24, identity=0, groups=(2, 2), scale=0.8, shared=16)),
                    _fol_layer("latent_attention", _fol_latent(3, 24, 8, 20, 40, 24, scale=0.2))]}
# latent attention first; a router without groups, identity experts or a shared expert that
# takes one expert; a state space layer without a feed-forward, a group a head, one part in
# its norm; a window of seven, no grouping of heads, values larger than keys; two identity
# experts among six outputs with one group of two kept; taps of four and of two
FOL_B = {"architecture": "Folivik", "vocab": 211, "width": 48, "norm": {"eps": 1e-6},
         "layers": [_fol_layer("latent_attention", _fol_latent(2, 16, 16, 16, 24, 16, base=500.0),
                               _fol_moe(5, 1, 40)),
                    _fol_layer("mamba2", _fol_mamba(3, 3, 8, 8, 4, 1)),
                    _fol_layer("attention", _fol_attn(3, 3, 24, 40, 7),
                               _fol_moe(4, 2, 16, identity=2, groups=(2, 1), scale=2.5, shared=56)),
                    _fol_layer("mamba2", _fol_mamba(2, 1, 40, 12, 2, 4),
                               _fol_moe(3, 3, 8, identity=1, groups=(1, 1), scale=1.0, shared=8))]}
# sizes that are multiples of two only: a width of 50, a vocabulary of 131, heads of 10 and 6,
# a state of 6; one head; a window of two; part of the rotated sizes turned; a convolution
# of one tap
FOL_C = {"architecture": "Folivik", "vocab": 131, "width": 50, "norm": {"eps": 1e-5},
         "layers": [_fol_layer("attention", _fol_attn(2, 1, 10, 6, 2, scale=0.5),
                               _fol_moe(2, 1, 6, identity=2, groups=(2, 2), scale=3.0, shared=10)),
                    _fol_layer("mamba2", _fol_mamba(2, 1, 6, 10, 1, 5), _fol_moe(7, 2, 10, shared=4)),
                    _fol_layer("latent_attention",
                               _fol_latent(1, 10, 6, 6, 14, 10, base=3000.0, dims=4),
                               _fol_moe(4, 4, 12, identity=0, groups=(4, 4), scale=0.5))]}
# wider, for bfloat16 and the tensor-core kernels: a latent of 192 with 32 rotated sizes,
# heads of 64 in a window of 48, a state of 64
FOL_D = {"architecture": "Folivik", "vocab": 500, "width": 192, "norm": {"eps": 1e-5},
         "layers": [_fol_layer("mamba2", _fol_mamba(6, 2, 64, 32, 4, 2),
                               _fol_moe(8, 2, 128, identity=2, groups=(5, 3), scale=2.0, shared=256)),
                    _fol_layer("latent_attention", _fol_latent(4, 64, 32, 64, 192, 96),
                               _fol_moe(6, 2, 96, identity=0, groups=(3, 2), scale=1.0, shared=128)),
                    _fol_layer("attention", _fol_attn(8, 4, 64, 64, 48),
                               _fol_moe(8, 3, 64, identity=1, groups=(3, 2), scale=1.5, shared=64)),
                    _fol_layer("mamba2", _fol_mamba(4, 4, 128, 48, 2, 1))]}

FOL = {
    "A": dict(raw=FOL_A, std=0.08, norm_std=0.1, page_size=16, seed=35),
    "B": dict(raw=FOL_B, std=0.1, norm_std=0.1, page_size=4, seed=36),
    "C": dict(raw=FOL_C, std=0.12, norm_std=0.1, page_size=8, seed=37),
    "D": dict(raw=FOL_D, std=0.05, norm_std=0.05, page_size=16, seed=38),
}


def make_folivik_dir(tmp_path, which, dtype=torch.float32, raw=None, tweak=None, tag="") -> str:
    """A folder with config.json and random weights of a configuration of this design;
    ``tweak(w)`` may change the tensors (a name -> tensor dictionary) before they are written."""
    from binfer_b200.config import FolivikConfig
    from binfer_b200.parts.model import param_specs_for
    from binfer_b200.weights import random_tensors, save_file
    t = FOL[which]
    raw = raw or t["raw"]
    cfg = FolivikConfig.from_dict(raw)
    d = os.path.join(str(tmp_path), f"fol_{which}{tag}_{str(dtype).split('.')[-1]}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    w = random_tensors(param_specs_for(cfg.to_spec()), t["seed"], t["std"], t["norm_std"], dtype)
    # corrections that decide choices now and then, some of them below minus the scores
    for n, x in w.items():
        if n.endswith(".correction"):
            g = torch.Generator().manual_seed(len(n) + x.numel())
            x.copy_((torch.randn(x.shape, generator=g) * 0.15 - 0.1).to(x.dtype))
    if tweak is not None:
        tweak(w)
    save_file(w, os.path.join(d, "model.safetensors"))
    return d
