"""Small Bilurax models for the tests: configurations that differ in every size and option, random weights whose
scales make every mechanism matter, and model folders written from them.

The weights are drawn in float32 and rounded to bfloat16 values, so the engine in either compute type and the
plain implementation (tests/plain_bilurax.py, in float64) start from the same numbers.

Routers.  A token's experts are the largest of a handful of scores, and two of them are now and then closer than
the rounding of a bfloat16 run moves them; the token then takes another expert and its logits land elsewhere, which
says nothing about the engine.  So `make_weights(..., decisive_router=True)` spreads the corrections far apart and
shrinks the router's matrix: the choice of groups and experts is then the same with either rounding (the weights of
the chosen experts still depend on the token).  The float32 tests use ordinary routers, whose choices change from
token to token.
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Dict, List, Optional

import numpy as np
import torch


def attention(heads, kv_heads, dim, vdim, chunk, softcap=15.0, scale=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
                      "scale": scale if scale is not None else dim ** -0.5, "softcap": softcap}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=1, keep=1, scale=1.0, limit=3.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}


def layer(mixer: dict, mlp: Optional[dict]) -> dict:
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    return out


def _config(vocab, width, layers, eps=1e-5, logit_softcap=25.0, embedding_scale=1.0, loop=None):
    c = {"architecture": "Bilurax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_softcap": logit_softcap,
         "embedding": {"scale": embedding_scale}, "layers": layers}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# A: a looped span in the middle (layers 1 and 2, twice), grouped-query heads of 32 (two query heads a key/value head),
# chunks of 24 and of 40 positions, all three feed-forwards, three groups of which two stay
CONFIG_A = _config(101, 64, [
    layer(attention(4, 2, 32, 32, 24), dense(96)),
    layer(attention(4, 2, 32, 32, 40), moe(6, 2, 24, groups=3, keep=2, scale=1.5)),
    layer(attention(2, 1, 16, 48, 24, softcap=6.0), None),
    layer(attention(4, 4, 16, 16, 1000), moe(4, 1, 40, groups=1, keep=1, scale=0.75, limit=1.0)),
], eps=1e-5, logit_softcap=12.0, embedding_scale=3.0, loop=(1, 3, 2))

# B: no loop; a width that is no multiple of 8 (the bfloat16 products then take the kernel for odd sizes); head
# sizes that divide by nothing (20 and 12: pages of 32 with zeros behind both); one head; chunks of 7 and of 1
# (a token sees itself alone); every expert chosen; groups of one expert
CONFIG_B = _config(77, 100, [
    layer(attention(1, 1, 20, 12, 7), moe(5, 5, 12, groups=1, keep=1, scale=2.5)),
    layer(attention(5, 5, 12, 20, 1), dense(52)),
    layer(attention(6, 2, 8, 8, 33, softcap=50.0), moe(6, 2, 20, groups=6, keep=3, scale=1.0, limit=0.5)),
], eps=1e-6, logit_softcap=40.0, embedding_scale=0.5)

# C: the whole stack looped three times; eight query heads on one key/value head with heads of 64 and values of 128
# (pages of 128: the decode kernels' widest rows); heads of 144 (beyond the tensor-core attention kernels); many experts
CONFIG_C = _config(311, 128, [
    layer(attention(8, 1, 64, 128, 48), moe(32, 4, 64, groups=4, keep=2, scale=2.0)),
    layer(attention(2, 2, 144, 16, 64), dense(256)),
], eps=1e-5, logit_softcap=30.0, embedding_scale=8.0, loop=(0, 2, 3))

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}


def tensor_shapes(config: dict) -> Dict[str, List[int]]:
    """Every tensor of a model of this configuration, by its name in the weight file."""
    w = config["width"]
    out = {"embed": [config["vocab"], w], "final.norm": [w]}
    if config.get("loop"):
        out["loop.step"] = [config["loop"]["times"], w]
    for i, l in enumerate(config["layers"]):
        p = f"l{i}."
        out[p + "norm1"] = [w]
        out[p + "shift"] = [w]
        m, x = l["mixer"], p + "mix."
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({x + "q": [H * d, w], x + "q.b": [H * d], x + "k": [G * d, w], x + "k.b": [G * d], x + "v": [G * e, w],
                    x + "v.b": [G * e], x + "q.norm": [H * d], x + "k.norm": [G * d], x + "temp": [H], x + "o": [w, H * e],
                    x + "o.b": [w]})
        mlp = l.get("mlp")
        if mlp:
            out[p + "norm2"] = [w]
            if mlp["kind"] == "dense":
                out.update({p + "mlp.up": [mlp["ff"], w], p + "mlp.down": [w, mlp["ff"]]})
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                out.update({p + "mlp.router": [E, w], p + "mlp.correction": [E]})
                for k in range(E):
                    out.update({f"{p}mlp.e{k}.gate": [ff, w], f"{p}mlp.e{k}.up": [ff, w], f"{p}mlp.e{k}.down": [w, ff]})
    return out


def make_weights(config: dict, seed: int, decisive_router: bool = False) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    groups_of = {}
    for i, l in enumerate(config["layers"]):
        if l.get("mlp") and l["mlp"]["kind"] == "moe":
            groups_of[f"l{i}.mlp.correction"] = l["mlp"]["router"]["groups"]["count"]
    for name, shape in tensor_shapes(config).items():
        last = name.split(".")[-1]
        n = lambda std=1.0, mean=0.0: mean + std * torch.randn(shape, generator=g)
        if name == "embed":
            t = n()
        elif name == "loop.step":
            t = n(0.5)
        elif last in ("norm1", "norm2") or name == "final.norm" or name.endswith("q.norm") or name.endswith("k.norm"):
            t = n(0.2, 1.0)
        elif last == "shift":
            t = torch.rand(shape, generator=g)                   # between "this token" and "the token before"
        elif last == "temp":
            t = n(0.3, 1.5)
        elif last == "b":                                         # biases of the projections
            t = n(0.3)
        elif last == "correction":
            if decisive_router:
                # far apart, and so that whole groups are far apart too: expert e of group j gets 3 (rank of j) + 0.3 (rank in j)
                count = groups_of[name]
                per = shape[0] // count
                gr = torch.randperm(count, generator=g).to(torch.float32)
                t = torch.cat([3.0 * gr[j] + 0.3 * torch.randperm(per, generator=g).to(torch.float32) for j in range(count)])
            else:
                t = n(0.3)
        elif last == "router":
            t = n((0.05 if decisive_router else 3.0) / math.sqrt(shape[1]))
        elif last == "down" and ".mlp.e" in name:
            t = n(2.0 / math.sqrt(shape[1]))
        elif len(shape) == 2:
            t = n(1.2 / math.sqrt(shape[1]))
        else:
            raise ValueError(name)
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def write_model(config: dict, weights: Dict[str, torch.Tensor], path: str, store=torch.bfloat16) -> str:
    from sandyrt_b200.weights.safetensors import write_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
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
