"""Small Tifepel models for the tests: configurations that differ in every size and option, random weights whose
scales make every mechanism matter, and model folders written from them.

The weights are drawn in float32 and rounded to bfloat16 values, so the engine in either compute type and the
plain implementation (tests/plain_tifepel.py, in float64) start from the same numbers.

Routers.  A token's experts are the largest of a handful of choice scores, and two of them are now and then closer
than the rounding of a bfloat16 run moves them; the token then takes another expert and its logits land elsewhere,
which says nothing about the engine.  So `make_weights(..., decisive_router=True)` spreads the corrections a whole
score apart (softmax scores lie in 0 .. 1) and shrinks the router's matrix: the choice is then the same with either
rounding (the weights of the chosen experts still depend on the token).  The float32 tests use ordinary routers,
whose choices change from token to token.
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Dict, List, Optional

import numpy as np
import torch


def attention(heads, kv_heads, dim, vdim, rows, far, every=16, coef=0.5, scale=None):
    """`rows`: the bias table's rows (the weight file decides; the configuration states it for random weights)."""
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "bias_max": far, "bias_rows": rows,
                      "q_temp": {"coef": coef, "every": every}, "scale": scale if scale is not None else dim ** -0.5}}


def mamba2(heads, groups, state, vdim, conv, norm_groups):
    return {"type": "mamba2",
            "mixer": {"heads": heads, "groups": groups, "state": state, "vdim": vdim, "conv": conv, "norm_groups": norm_groups}}


def moe(experts, identity, top, ff, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top},
            "shared": {"ff": shared} if shared else None}


def layer(mixer: dict, mlp: Optional[dict]) -> dict:
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    return out


def _config(vocab, width, layers, streams=2, taps=4, eps=1e-5, max_positions=512, bigram=(31, 7, 3), loop=None):
    c = {"architecture": "Tifepel", "vocab": vocab, "width": width, "max_positions": max_positions, "streams": streams,
         "norm": {"eps": eps}, "canon": {"taps": taps},
         "embedding": {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}, "layers": layers}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# A: three streams, two taps, a looped span in the middle (layers 1 and 2, twice); grouped-query heads with values
# wider than keys; a state of 16 with three taps; a layer without a feed-forward; more identity experts than chosen
CONFIG_A = _config(101, 64, [
    layer(attention(4, 2, 16, 32, rows=8, far=40, every=5, coef=0.7), moe(6, 2, 3, 24, shared=40)),
    layer(mamba2(4, 2, 16, 8, conv=3, norm_groups=1), moe(4, 4, 2, 16, shared=16)),
    layer(attention(2, 1, 24, 8, rows=6, far=17, every=64, coef=0.25, scale=0.3), None),
    layer(mamba2(6, 3, 24, 16, conv=2, norm_groups=4), moe(5, 1, 5, 8)),
], streams=3, taps=2, eps=1e-5, bigram=(31, 7, 3), loop=(1, 3, 2))

# B: one stream, one tap (the convolution is a factor), no loop; a width that is no multiple of 8 (the bfloat16 products
# then take the kernel for odd sizes); sizes that divide by nothing (a state of 40, values of 12, heads of 12 and 20);
# as many groups as heads, one tap in the mixer's convolution; no identity experts, every expert chosen, no shared one
CONFIG_B = _config(77, 100, [
    layer(mamba2(5, 5, 40, 12, conv=1, norm_groups=5), moe(3, 0, 3, 12)),
    layer(attention(5, 5, 12, 20, rows=4, far=9, every=1, coef=1.0), moe(4, 0, 1, 20, shared=28)),
    layer(mamba2(2, 1, 7, 30, conv=4, norm_groups=3), None),
], streams=1, taps=1, eps=1e-6, bigram=(5, 1, 1))

# C: four streams, four taps, the whole stack looped three times; eight query heads of 64 on one key/value head; a state
# of 128 with values of 64 (the recurrence's widest common shape); many experts, a third of them identities
CONFIG_C = _config(311, 128, [
    layer(attention(8, 1, 64, 64, rows=32, far=100, every=32, coef=0.5), moe(20, 12, 6, 32, shared=64)),
    layer(mamba2(2, 1, 128, 64, conv=4, norm_groups=2), moe(8, 8, 4, 48, shared=16)),
], streams=4, taps=4, eps=1e-5, bigram=(499, 131, 19), loop=(0, 2, 3))

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}


def tensor_shapes(config: dict) -> Dict[str, List[int]]:
    """Every tensor of a model of this configuration, by its name in the weight file."""
    w, S, taps = config["width"], config["streams"], config["canon"]["taps"]
    out = {"embed": [config["vocab"], w], "bigram": [config["embedding"]["bigram"]["buckets"] + 1, w],
           "pos": [config["max_positions"], w], "final.norm": [w], "head": [config["vocab"], w]}
    for i, l in enumerate(config["layers"]):
        p = f"l{i}."
        for q in ("1", "2") if l.get("mlp") else ("1",):
            out.update({p + "norm" + q: [w], p + f"hc{q}.in": [S], p + f"hc{q}.out": [S], p + f"hc{q}.mix": [S, S],
                        p + "canon" + q: [w, taps], p + "rg" + q: [w, w], p + f"rg{q}.b": [w]})
        m, x = l["mixer"], p + "mix."
        if l["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({x + "q": [H * d, w], x + "k": [G * d, w], x + "v": [G * e, w], x + "o": [w, H * e], x + "rel": [m["bias_rows"], H]})
        else:
            H, G, N, P = m["heads"], m["groups"], m["state"], m["vdim"]
            inner, ch = H * P, H * P + 2 * G * N
            out.update({x + "in": [inner + ch + H, w], x + "conv": [ch, m["conv"]], x + "conv.b": [ch], x + "dt_bias": [H],
                        x + "A_log": [H], x + "D": [H], x + "norm": [inner], x + "o": [w, inner]})
        mlp = l.get("mlp")
        if mlp:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            out.update({p + "mlp.router": [r["experts"] + r["identity"], w], p + "mlp.correction": [r["experts"] + r["identity"]]})
            for k in range(r["experts"]):
                out.update({f"{p}mlp.e{k}.gate": [ff, w], f"{p}mlp.e{k}.up": [ff, w], f"{p}mlp.e{k}.down": [w, ff]})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": [sf, w], p + "mlp.shared.up": [sf, w], p + "mlp.shared.down": [w, sf]})
    return out


def make_weights(config: dict, seed: int, decisive_router: bool = False) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    S = config["streams"]
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.split(".")[-1]
        n = lambda std=1.0, mean=0.0: mean + std * torch.randn(shape, generator=g)
        if name in ("embed", "bigram"):
            t = n(0.7)
        elif name == "pos":
            t = n(0.5)
        elif name == "head":
            t = n(1.0 / math.sqrt(shape[1]))
        elif last in ("norm1", "norm2") or name == "final.norm" or name.endswith("mix.norm"):
            t = n(0.2, 1.0)
        elif name.endswith(".in") and ".hc" in name:
            t = n(0.3, 1.0 / S)
        elif name.endswith(".out") and ".hc" in name:
            t = n(0.3, 1.0)
        elif name.endswith(".mix") and ".hc" in name:
            t = torch.eye(S) + n(0.25)
        elif last in ("canon1", "canon2"):
            t = n(0.4)
        elif last in ("rg1", "rg2"):
            t = n(1.5 / math.sqrt(shape[1]))
        elif last == "b" and ".rg" in name:
            t = n(1.0)
        elif last == "rel":
            t = n(1.0)
        elif last == "conv":
            t = n(0.5)
        elif last == "b" and name.endswith("conv.b"):
            t = n(0.2)
        elif last == "dt_bias":
            t = n(1.0, -1.5)
        elif last == "A_log":
            t = torch.log(0.3 + 3.0 * torch.rand(shape, generator=g))
        elif last == "D":
            t = n(0.3, 1.0)
        elif last == "correction":
            if decisive_router:
                t = 1.0 * torch.randperm(shape[0], generator=g).to(torch.float32)
            else:
                t = n(0.05)
        elif last == "router":
            t = n((0.05 if decisive_router else 3.0) / math.sqrt(shape[1]))
        elif last == "down" and ".mlp." in name:
            t = n(2.0 / math.sqrt(shape[1]))
        elif len(shape) == 2:
            t = n(1.2 / math.sqrt(shape[1]))
        else:
            raise ValueError(name)
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def write_model(config: dict, weights: Dict[str, torch.Tensor], path: str, store=torch.bfloat16, drop_bias_rows: bool = True) -> str:
    """`drop_bias_rows`: the configuration on disk leaves the bias tables' row counts to the weight file."""
    from sandyrt_b200.weights.safetensors import write_safetensors

    os.makedirs(path, exist_ok=True)
    on_disk = copy.deepcopy(config)
    if drop_bias_rows:
        for l in on_disk["layers"]:
            l["mixer"].pop("bias_rows", None)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(on_disk, f, indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.to(store) for k, v in weights.items()})
    return path


def rel_error(got: np.ndarray, want: np.ndarray) -> float:
    """Largest over the rows of: RMS over the vocabulary of the difference (mean taken off) over the RMS of the
    wanted logits (mean taken off)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float((np.sqrt((d ** 2).mean(-1)) / np.sqrt((w ** 2).mean(-1))).max())
