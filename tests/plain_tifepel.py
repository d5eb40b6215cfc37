"""Tifepel, plainly: whole sequences in float64, no cache, one function per mechanism.

This is what the engine is compared with.  It shares no code with the engine: it reads a configuration (the
dictionary of config.json) and a dictionary of tensors by their names in the weight file, and walks a whole token
sequence through every layer with ordinary tensor arithmetic.

The design, in this file's notation (W x means W @ x with W stored [out, in]; rms(x) = sqrt(mean(x^2) + eps);
ln(x, g) = (x - mean) / sqrt(var + eps) * g with the biased variance):

  embedding     e_t = E[tok_t] + Bg[(tok_{t-1} a + tok_t b) mod n] + P[t]; the first token reads Bg[n]
  streams       X_1 .. X_S all start as e; the logits read ln(sum_s X_s, g_final)
  sublayer q    u = sum_s in_q[s] X_s;  h = ln(u, g_q);  c = h + conv_q(h) (causal, per channel, `taps` taps)
                y = f_q(c) * sigmoid(R_q h + r_q);  X_t <- sum_s mix_q[s, t] X_s + out_q[t] y
  attention     q, k = unit root mean square per head; q_i *= 1 + coef ln(floor((i + 1) / every) + 1)
                s_ij = (q_i . k_j) scale + rel[bucket(i - j), head], j <= i; softmax; W_o
                bucket(n) = n below half = B / 2, else min(B - 1, half + floor(ln(n / half) / ln(D / half) (B - half)))
  mamba2        [z | x | B | C | dt] = W_in c; (x, B, C) <- silu(causal conv + bias); dt <- softplus(dt + dt_bias)
                S_t = exp(-exp(A_log) dt) S_{t-1} + dt B_t x_t^T; y_t = S_t^T C_t + D x_t per head
                y <- y silu(z), unit root mean square in `norm_groups` equal parts, times a gain; W_o
  feed-forward  scores s = softmax(W_r h) over routed + identity experts; the `top` largest s + correction are chosen,
                weighted by s itself; expert = W_d (silu(W_g h) (W_u h)), identity expert = h; a shared expert is added

`forward_rounded` does the same with the operands and results of the matrix products rounded to bfloat16 values
(what a bfloat16 engine must do at least), for the tests' bfloat16 bounds.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch

F = torch.float64


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
        return y if keep else _bf16(y)          # keep: a product whose result stays 32-bit

    def round(self, t: torch.Tensor) -> torch.Tensor:
        return _bf16(t) if self.rounded else t


def layer_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * gain


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def causal_conv(h: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """out_t = sum_j taps[:, j] h_(t - n + 1 + j), zeros before the start; taps [channels, n]."""
    n = taps.shape[1]
    out = torch.zeros_like(h)
    for j in range(n):
        back = n - 1 - j
        if back == 0:
            out += h * taps[:, j]
        elif back < h.shape[0]:
            out[back:] += h[:-back] * taps[:, j]
    return out


def embedding(config: dict, w: Dict[str, torch.Tensor], ids) -> torch.Tensor:
    b = config["embedding"]["bigram"]
    ids = list(ids)
    rows = [b["buckets"]] + [(ids[t - 1] * b["mul_prev"] + ids[t] * b["mul_cur"]) % b["buckets"] for t in range(1, len(ids))]
    return w["embed"][torch.tensor(ids)] + w["bigram"][torch.tensor(rows)] + w["pos"][: len(ids)]


def distance_bucket(n: int, rows: int, far: float) -> int:
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def attention(m: dict, eps: float, w: Dict[str, torch.Tensor], p: str, c: torch.Tensor, mm: Products) -> torch.Tensor:
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = c.shape[0]
    q = unit_rms(mm(c, w[p + "q"]).view(n, H, d), eps)
    k = unit_rms(mm(c, w[p + "k"]).view(n, G, d), eps)
    v = mm(c, w[p + "v"]).view(n, G, e)
    pos = torch.arange(n)
    temp = 1.0 + m["q_temp"]["coef"] * torch.log(torch.div(pos + 1, m["q_temp"]["every"], rounding_mode="floor").to(F) + 1.0)
    q = mm.round(q * temp[:, None, None])
    k = mm.round(k)
    rel = w[p + "rel"]
    bucket = torch.tensor([distance_bucket(i, rel.shape[0], m["bias_max"]) for i in range(n)])
    dist = (pos[:, None] - pos[None, :]).clamp(min=0)
    see = pos[None, :] <= pos[:, None]
    out = torch.zeros(n, H, e, dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].t()) * m["scale"] + rel[:, h][bucket[dist]]
        s = s.masked_fill(~see, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return mm(mm.round(out).reshape(n, H * e), w[p + "o"], keep=True)


def mamba2(m: dict, eps: float, w: Dict[str, torch.Tensor], p: str, c: torch.Tensor, mm: Products) -> torch.Tensor:
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    n = c.shape[0]
    proj = mm(c, w[p + "in"], keep=True)
    z = mm.round(proj[:, :inner])
    xbc = mm.round(proj[:, inner: 2 * inner + 2 * G * N])
    dt = proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"]) + w[p + "conv.b"])
    x = xbc[:, :inner].view(n, H, P)
    B = xbc[:, inner: inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"], threshold=1e9)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros(n, H, P, dtype=F)
    S = torch.zeros(H, N, P, dtype=F)
    group = torch.arange(H) // (H // G)
    for t in range(n):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t][group][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, C[t][group]) + w[p + "D"][:, None] * x[t]
    y = y.reshape(n, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(n, parts, inner // parts), eps).reshape(n, inner) * w[p + "norm"]
    return mm(y, w[p + "o"], keep=True)


def gated_expert(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, mm: Products) -> torch.Tensor:
    a = silu(mm(h, w[p + "gate"])) * mm(h, w[p + "up"])
    return mm(a, w[p + "down"], keep=True)


def route(r: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, mm: Products):
    """(chosen experts [T, top], their weights [T, top], the margin by which the choice was made [T])."""
    s = torch.softmax(mm(h, w[p + "router"], keep=True), -1)
    ranked = (s + w[p + "correction"]).sort(dim=-1, descending=True, stable=True)
    top = r["top"]
    chosen = ranked.indices[:, :top]
    margin = torch.full((h.shape[0],), math.inf, dtype=F)
    if top < s.shape[1]:
        margin = ranked.values[:, top - 1] - ranked.values[:, top]
    return chosen, s.gather(1, chosen), margin


def moe(mlp: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, mm: Products) -> torch.Tensor:
    r = mlp["router"]
    chosen, weights, _ = route(r, w, p, h, mm)
    out = torch.zeros_like(h)
    for k in range(r["experts"] + r["identity"]):
        hit = chosen == k
        rows = hit.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        y = gated_expert(w, f"{p}e{k}.", h[rows], mm) if k < r["experts"] else mm.round(h[rows])
        out[rows] += (weights[rows] * hit[rows]).sum(-1, keepdim=True) * y
    if mlp.get("shared"):
        out = out + gated_expert(w, p + "shared.", h, mm)
    return out


def run_order(config: dict) -> List[int]:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], n))


def sublayer(config: dict, w: Dict[str, torch.Tensor], p: str, q: int, X: torch.Tensor, f, mm: Products) -> torch.Tensor:
    """X [streams, T, width] -> the streams after sublayer q of the layer whose tensors start with p."""
    eps = config["norm"]["eps"]
    u = torch.einsum("s,stw->tw", w[f"{p}hc{q}.in"], X)
    h = mm.round(layer_norm(u, w[f"{p}norm{q}"], eps))
    c = h + causal_conv(h, w[f"{p}canon{q}"])
    y = f(c) * torch.sigmoid(mm(h, w[f"{p}rg{q}"], w[f"{p}rg{q}.b"], keep=True))
    return torch.einsum("st,sxw->txw", w[f"{p}hc{q}.mix"], X) + w[f"{p}hc{q}.out"][:, None, None] * y[None]


def forward(config: dict, weights: Dict[str, torch.Tensor], ids, rounded: bool = False,
            after_layer: Optional[Callable[[int, torch.Tensor], None]] = None,
            only: Optional[Callable[[int, int], bool]] = None) -> torch.Tensor:
    """Logits [len(ids), vocab] of a whole sequence.  `only(layer, q)` false leaves sublayer q of a layer out."""
    w = {k: v.to(F) for k, v in weights.items()}
    mm = Products(rounded)
    eps = config["norm"]["eps"]
    e = embedding(config, w, ids)
    X = e[None].repeat(config["streams"], 1, 1)
    for run, i in enumerate(run_order(config)):
        l, p = config["layers"][i], f"l{i}."
        mixer = attention if l["type"] == "attention" else mamba2
        if only is None or only(i, 1):
            X = sublayer(config, w, p, 1, X, lambda c: mixer(l["mixer"], eps, w, p + "mix.", c, mm), mm)
        if l.get("mlp") and (only is None or only(i, 2)):
            X = sublayer(config, w, p, 2, X, lambda c: moe(l["mlp"], w, p + "mlp.", c, mm), mm)
        if after_layer:
            after_layer(run, X.sum(0))
    y = layer_norm(X.sum(0), w["final.norm"], eps)
    return mm(y, w["head"], keep=True)


def forward_rounded(config: dict, weights: Dict[str, torch.Tensor], ids) -> torch.Tensor:
    return forward(config, weights, ids, rounded=True)


def router_margin(config: dict, weights: Dict[str, torch.Tensor], ids) -> float:
    """The smallest gap by which any token's choice of experts was made, over all feed-forwards: a run whose rounding
    moves a choice score by less than this chooses the same experts."""
    w = {k: v.to(F) for k, v in weights.items()}
    mm = Products(False)
    eps = config["norm"]["eps"]
    smallest = [math.inf]
    X = embedding(config, w, ids)[None].repeat(config["streams"], 1, 1)
    for i in run_order(config):
        l, p = config["layers"][i], f"l{i}."
        mixer = attention if l["type"] == "attention" else mamba2
        X = sublayer(config, w, p, 1, X, lambda c: mixer(l["mixer"], eps, w, p + "mix.", c, mm), mm)
        if l.get("mlp"):
            def ff(c):
                smallest[0] = min(smallest[0], float(route(l["mlp"]["router"], w, p + "mlp.", c, mm)[2].min()))
                return moe(l["mlp"], w, p + "mlp.", c, mm)
            X = sublayer(config, w, p, 2, X, ff, mm)
    return smallest[0]


def generate_greedy(config: dict, weights: Dict[str, torch.Tensor], prompt, n: int) -> List[int]:
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(forward(config, weights, ids)[-1].argmax()))
    return ids[len(prompt):]
