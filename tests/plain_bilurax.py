"""Bilurax, plainly: whole sequences in float64, no cache, one function per mechanism.

This is what the engine is compared with.  It shares no code with the engine: it reads a configuration (the
dictionary of config.json) and a dictionary of tensors by their names in the weight file, and walks a whole token
sequence through every layer with ordinary tensor arithmetic.

The design, in this file's notation (W x means W @ x with W stored [out, in]; rms(x) = sqrt(mean(x^2) + eps)):

  x_t   = E[token_t] * embedding.scale
  before pass p of the looped span: x += x_at_embedding (p > 0), then x += loop.step[p]
  layer: h = norm1(x) = x / rms(x) * g1
         token shift   u_t = h_t + (h_{t-1} - h_t) * shift,  h_{-1} = 0
         attention     q = Wq u + bq, k = Wk u + bk, v = Wv u + bv
                       q <- q / rms(q) * gq  over the whole row, k likewise; each head of v <- v / rms(v)
                       s_ij = cap * tanh((q_i . k_j) * scale * temp_head / cap), j <= i and floor(i / C) == floor(j / C)
                       o = softmax(s) v; x += Wo [heads] + bo
         feed-forward  n = norm2(x);  dense: x += Wd relu(Wu n)^2
                       routed: s = sigmoid(Wr n), choice c = s + correction; groups of neighbours, a group's score the
                       sum of its two largest c, the `keep` best groups stay; the `top` largest c among them are
                       chosen; weights s_chosen / (sum + 1e-20) * router.scale; expert: g = min(Wg n, L),
                       u = clamp(Wu n, -L, L), y = Wd (g * sigmoid(1.702 g) * (u + 1))
  logits = lc * tanh((E normf(x)) / lc)

`forward_rounded` does the same with the operands and results of the matrix products rounded to bfloat16 values
(what a bfloat16 engine must do at least), for the tests' bfloat16 bounds.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch

F = torch.float64
GLU_ALPHA = 1.702
WEIGHT_EPS = 1e-20


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).to(torch.bfloat16).to(F)


class Products:
    """y = W x, exactly or with operands and result rounded to bfloat16 values."""

    def __init__(self, rounded: bool):
        self.rounded = rounded

    def __call__(self, x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, keep: bool = False) -> torch.Tensor:
        if not self.rounded:
            y = x @ w.t()
            return y + b if b is not None else y
        y = _bf16(x) @ w.t()
        if b is not None:
            y = y + b
        return y if keep else _bf16(y)          # keep: a product whose result stays 32-bit (router logits, the stream)


def rms_norm(x: torch.Tensor, gain: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y * gain if gain is not None else y


def token_shift(h: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    before = torch.zeros_like(h)
    before[1:] = h[:-1]
    return h + (before - h) * mix


def visible(n: int, chunk: int) -> torch.Tensor:
    """[i, j] true where query i sees key j: not later, and in the same chunk of positions."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))


def attention(m: dict, eps: float, w: Dict[str, torch.Tensor], p: str, u: torch.Tensor, mm: Products) -> torch.Tensor:
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = u.shape[0]
    q = mm(u, w[p + "q"], w[p + "q.b"])
    k = mm(u, w[p + "k"], w[p + "k.b"])
    v = mm(u, w[p + "v"], w[p + "v.b"])
    q = rms_norm(q, w[p + "q.norm"], eps).view(n, H, d)
    k = rms_norm(k, w[p + "k.norm"], eps).view(n, G, d)
    v = rms_norm(v.view(n, G, e), None, eps)
    if mm.rounded:                              # what the cache and the query matrix hold
        q = _bf16(q * w[p + "temp"][None, :, None])
        k, v = _bf16(k), _bf16(v)
    else:
        q = q * w[p + "temp"][None, :, None]
    see = visible(n, m["mask"]["size"])
    out = torch.zeros(n, H, e, dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].t()) * m["scale"]
        s = m["softcap"] * torch.tanh(s / m["softcap"])
        s = s.masked_fill(~see, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    if mm.rounded:
        out = _bf16(out)
    return mm(out.reshape(n, H * e), w[p + "o"], w[p + "o.b"], keep=True)


def dense_ff(w: Dict[str, torch.Tensor], p: str, n: torch.Tensor, mm: Products) -> torch.Tensor:
    a = torch.relu(mm(n, w[p + "up"], keep=True)) ** 2
    return mm(_bf16(a) if mm.rounded else a, w[p + "down"], keep=True)


def route(r: dict, w: Dict[str, torch.Tensor], p: str, n: torch.Tensor, mm: Products):
    """(chosen experts [T, top], their weights [T, top], the margin by which the choice was made [T])."""
    E, top, count, keep = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
    s = torch.sigmoid(mm(n, w[p + "router"], keep=True))
    c = s + w[p + "correction"]
    per = E // count
    group_score = c.view(-1, count, per).topk(min(2, per), -1).values.sum(-1)
    order = group_score.argsort(dim=-1, descending=True, stable=True)
    kept = torch.zeros_like(group_score, dtype=torch.bool)
    kept.scatter_(1, order[:, :keep], True)
    c_in = c.masked_fill(~kept.repeat_interleave(per, dim=1), -math.inf)
    ranked = c_in.sort(dim=-1, descending=True, stable=True)
    chosen = ranked.indices[:, :top]
    margin = torch.full((n.shape[0],), math.inf, dtype=F)
    if top < per * keep:
        margin = ranked.values[:, top - 1] - ranked.values[:, top]
    if keep < count:
        gs = group_score.sort(-1, descending=True).values
        margin = torch.minimum(margin, gs[:, keep - 1] - gs[:, keep])
    picked = s.gather(1, chosen)
    weights = picked / (picked.sum(-1, keepdim=True) + WEIGHT_EPS) * r["scale"]
    return chosen, weights, margin


def expert(limit: float, w: Dict[str, torch.Tensor], p: str, n: torch.Tensor, mm: Products) -> torch.Tensor:
    g = torch.clamp(mm(n, w[p + "gate"]), max=limit)
    u = torch.clamp(mm(n, w[p + "up"]), -limit, limit)
    y = g * torch.sigmoid(GLU_ALPHA * g) * (u + 1.0)
    return mm(_bf16(y) if mm.rounded else y, w[p + "down"], keep=True)


def routed_ff(mlp: dict, w: Dict[str, torch.Tensor], p: str, n: torch.Tensor, mm: Products) -> torch.Tensor:
    chosen, weights, _ = route(mlp["router"], w, p, n, mm)
    out = torch.zeros_like(n)
    for k in range(mlp["router"]["experts"]):
        hit = (chosen == k)
        rows = hit.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        y = expert(mlp["expert"]["limit"], w, f"{p}e{k}.", n[rows], mm)
        out[rows] += (weights[rows] * hit[rows]).sum(-1, keepdim=True) * y
    return out


def run_order(config: dict) -> List[tuple]:
    """(layer, pass of the looped span that starts here or None) for every layer run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        out += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return out + [(i, None) for i in range(loop["stop"], n)]


def forward(config: dict, weights: Dict[str, torch.Tensor], ids, rounded: bool = False,
            after_layer: Optional[Callable[[int, torch.Tensor], None]] = None) -> torch.Tensor:
    """Logits [len(ids), vocab] of a whole sequence."""
    w = {k: v.to(F) for k, v in weights.items()}
    mm = Products(rounded)
    eps = config["norm"]["eps"]
    x0 = w["embed"][torch.tensor(list(ids))] * config["embedding"]["scale"]
    x = x0.clone()
    for run, (i, entering) in enumerate(run_order(config)):
        if entering is not None:
            if entering > 0:
                x = x + x0
            x = x + w["loop.step"][entering]
        l, p = config["layers"][i], f"l{i}."
        u = token_shift(rms_norm(x, w[p + "norm1"], eps), w[p + "shift"])
        x = x + attention(l["mixer"], eps, w, p + "mix.", u, mm)
        mlp = l.get("mlp")
        if mlp:
            n = rms_norm(x, w[p + "norm2"], eps)
            x = x + (dense_ff(w, p + "mlp.", n, mm) if mlp["kind"] == "dense" else routed_ff(mlp, w, p + "mlp.", n, mm))
        if after_layer:
            after_layer(run, x)
    y = rms_norm(x, w["final.norm"], eps)
    logits = mm(y, w["embed"], keep=True)
    cap = config["logit_softcap"]
    return cap * torch.tanh(logits / cap)


def forward_rounded(config: dict, weights: Dict[str, torch.Tensor], ids) -> torch.Tensor:
    return forward(config, weights, ids, rounded=True)


def router_margin(config: dict, weights: Dict[str, torch.Tensor], ids) -> float:
    """The smallest gap by which any token's choice of experts or of groups was made, over all routed layers: a
    run whose rounding moves a score by less than this chooses the same experts."""
    w = {k: v.to(F) for k, v in weights.items()}
    mm = Products(False)
    eps = config["norm"]["eps"]
    smallest = [math.inf]
    x0 = w["embed"][torch.tensor(list(ids))] * config["embedding"]["scale"]
    x = x0.clone()
    for i, entering in run_order(config):
        if entering is not None:
            x = x + (x0 if entering > 0 else 0) + w["loop.step"][entering]
        l, p = config["layers"][i], f"l{i}."
        u = token_shift(rms_norm(x, w[p + "norm1"], eps), w[p + "shift"])
        x = x + attention(l["mixer"], eps, w, p + "mix.", u, mm)
        mlp = l.get("mlp")
        if mlp:
            n = rms_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "moe":
                smallest[0] = min(smallest[0], float(route(mlp["router"], w, p + "mlp.", n, mm)[2].min()))
                x = x + routed_ff(mlp, w, p + "mlp.", n, mm)
            else:
                x = x + dense_ff(w, p + "mlp.", n, mm)
    return smallest[0]


def generate_greedy(config: dict, weights: Dict[str, torch.Tensor], prompt, n: int) -> List[int]:
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(forward(config, weights, ids)[-1].argmax()))
    return ids[len(prompt):]
