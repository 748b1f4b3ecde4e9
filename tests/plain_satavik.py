"""A plain, slow implementation of the Satavik design in float64 on the CPU, one function per mechanism, written from
the design's equations and sharing no code with the library. Tests compare the library's results with it.

Notation: h is a sublayer's input [tokens, width] of ONE sequence; `start` is the position of its first token; a layer's
cache is a dict with "k" [positions, kv_heads, 2, dim] (normed and rotated keys of both maps) and "v" [positions,
kv_heads, vdim], extended by the layer that owns it and only read by a layer that borrows it. Weights are applied as
W x (stored [out, in])."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x: [tokens, ..., dim]. Of the last dimension's first `dims` places, place i turns with place i + dims/2 by the
    angle position * base^(-2i/dims); the places behind pass unchanged."""
    out = x.clone()
    half = dims // 2
    shape = [-1] + [1] * (x.dim() - 2)
    for i in range(half):
        angle = positions.to(F64) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def capped(score: torch.Tensor, cap: float) -> torch.Tensor:
    """cap * tanh(score / cap)."""
    return cap * torch.tanh(score / cap)


def visible(i: int, chunk: int) -> range:
    """The positions that position i sees: those of its own chunk of `chunk` positions, up to itself."""
    return range((i // chunk) * chunk, i + 1)


def difference_weight(w: dict, diff: float) -> float:
    """exp(lq1 . lk1) - exp(lq2 . lk2) + diff: one number for the layer."""
    return math.exp(float(w["lq1"].double() @ w["lk1"].double())) - \
        math.exp(float(w["lq2"].double() @ w["lk2"].double())) + diff


def project_keys(w: dict, p: dict, h: torch.Tensor, start: int, eps: float, cache: dict) -> None:
    """Appends the normed, rotated keys of both maps and the values of h's tokens to `cache`."""
    n = h.shape[0]
    kv_heads, dim, vdim = p["kv_heads"], p["dim"], p["vdim"]
    positions = torch.arange(start, start + n)
    k = (h @ w["k"].T).view(n, kv_heads, 2, dim)
    k = rms(k, eps) * w["k.norm"]
    k = rotate_halves(k, positions, p["rot"]["dims"], p["rot"]["base"])
    v = (h @ w["v"].T).view(n, kv_heads, vdim)
    cache["k"] = k if "k" not in cache else torch.cat([cache["k"], k])
    cache["v"] = v if "v" not in cache else torch.cat([cache["v"], v])


def differential_attention(w: dict, p: dict, h: torch.Tensor, start: int, eps: float, cache: dict) -> torch.Tensor:
    """Two softmax maps per head over the same values, combined as a1 - lambda a2, the difference divided by its root
    mean square and scaled by 1 - diff, each head gated by a sigmoid, then W_o. `cache` already holds the keys and
    values of every position up to the last token of h (this layer's own, or another layer's)."""
    n = h.shape[0]
    heads, kv_heads, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    positions = torch.arange(start, start + n)
    q = (h @ w["q"].T).view(n, heads, 2, dim)
    q = rms(q, eps) * w["q.norm"]
    q = rotate_halves(q, positions, p["rot"]["dims"], p["rot"]["base"])
    lam = difference_weight(w, p["diff"])
    gate = sigmoid(h @ w["g"].T)  # [tokens, heads]
    out = torch.zeros(n, heads, vdim, dtype=F64)
    for t in range(n):
        seen = list(visible(start + t, p["mask"]["size"]))
        for head in range(heads):
            g = head // (heads // kv_heads)
            maps = []
            for m in range(2):
                scores = capped((cache["k"][seen, g, m] @ q[t, head, m]) * p["scale"], p["softcap"])
                maps.append(torch.softmax(scores, dim=0) @ cache["v"][seen, g])
            o = maps[0] - lam * maps[1]
            out[t, head] = rms(o, eps) * (1.0 - p["diff"]) * gate[t, head]
    return out.reshape(n, heads * vdim) @ w["o"].T


def clamped_expert(w: dict, prefix: str, h: torch.Tensor, limit: float) -> torch.Tensor:
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ w[prefix + "gate"].T, max=limit)
    u = torch.clamp(h @ w[prefix + "up"].T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].T


def route(w: dict, h: torch.Tensor, top: int) -> tuple[torch.Tensor, torch.Tensor]:
    """The `top` experts with the largest router logits of every token and their weights: the softmax over the chosen
    logits only. Returns (experts [tokens, top], weights [tokens, top])."""
    logits = h @ w["router"].T + w["router.b"]
    values, chosen = torch.topk(logits, top, dim=-1)
    return chosen, torch.softmax(values, dim=-1)


def mixture(w: dict, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    """The weighted sum of every token's chosen experts plus the shared expert, which runs for every token."""
    chosen, weights = route(w, h, mlp["router"]["top"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t].tolist(), weights[t]):
            out[t] += weight * clamped_expert(w, f"e{e}.", h[t:t + 1], mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        out = out + clamped_expert(w, "shared.", h, mlp["shared"]["limit"])
    return out


def sub(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t.double() for name, t in weights.items() if name.startswith(prefix)}


class PlainSatavik:
    """The whole model on one sequence, fed in pieces: `feed(tokens)` returns the logits of the piece's tokens
    [tokens, vocab] and, if asked, the stream after every layer."""

    def __init__(self, config: dict, weights: dict) -> None:
        self.config = config
        self.w = {name: t.double() for name, t in weights.items()}
        self.caches = [dict() for _ in config["layers"]]
        self.length = 0

    def feed(self, tokens, keep_layers: bool = False):
        c, w = self.config, self.w
        eps = c["norm"]["eps"]
        x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * c["embedding"]["scale"]
        kept = []
        for index, layer in enumerate(c["layers"]):
            mix, p = sub(w, f"l{index}.mix."), layer["mixer"]
            source = p.get("kv_from")
            if source is None:
                project_keys(mix, p, x, self.length, eps, self.caches[index])
                cache = self.caches[index]
            else:
                cache = self.caches[source]
            y = differential_attention(mix, p, x, self.length, eps, cache)
            x = x + rms(y, eps) * w[f"l{index}.norm1"]
            if layer.get("mlp") is not None:
                y = mixture(sub(w, f"l{index}.mlp."), layer["mlp"], x)
                x = x + rms(y, eps) * w[f"l{index}.norm2"]
            kept.append(x.clone())
        self.length += len(tokens)
        logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T
        return (logits, torch.stack(kept)) if keep_layers else logits


def forward(config: dict, weights: dict, tokens) -> torch.Tensor:
    """Logits [tokens, vocab] of one sequence run whole."""
    return PlainSatavik(config, weights).feed(list(tokens))
