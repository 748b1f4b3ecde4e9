"""A plain, slow implementation of the Tisalorn design in float64 on the CPU, one function per mechanism, written
from the design's equations and sharing no code with the library. Tests compare the library's results with it.

Notation: h is a mixer's or feed-forward's input [tokens, width]; all functions work on ONE sequence, token by
token where a recurrence is involved, and take and return their state explicitly so that a test can cut a prompt
anywhere. Weights are applied as W x (stored [out, in])."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(variance + eps) * w, the variance being the mean squared deviation; no bias."""
    mean = x.mean(dim=-1, keepdim=True)
    dev = x - mean
    return dev / torch.sqrt((dev * dev).mean(dim=-1, keepdim=True) + eps) * w


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x: [tokens, heads, dim]. The first `dims` dimensions of each head are rotated, dimension 2i paired with
    2i + 1, by the angle position * base^(-2i/dims); the rest pass unchanged."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(F64) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def softmax_attention(w: dict, p: dict, h: torch.Tensor, start: int, cache: dict) -> torch.Tensor:
    """Causal softmax attention whose values are the keys as projected (before rotation). `cache` holds "k"
    (rotated keys) and "v" of the positions before `start` and is extended. Returns W_o on the concatenated heads."""
    n = h.shape[0]
    heads, kv_heads, dim = p["heads"], p["kv_heads"], p["dim"]
    q = (h @ w["q"].T).view(n, heads, dim)
    k = (h @ w["k"].T).view(n, kv_heads, dim)
    v = k.clone()
    positions = torch.arange(start, start + n)
    q = rotate_interleaved(q, positions, p["rot"]["dims"], p["rot"]["base"])
    k = rotate_interleaved(k, positions, p["rot"]["dims"], p["rot"]["base"])
    cache["k"] = k if "k" not in cache else torch.cat([cache["k"], k])
    cache["v"] = v if "v" not in cache else torch.cat([cache["v"], v])
    out = torch.zeros(n, heads, dim, dtype=F64)
    for t in range(n):
        seen = start + t + 1
        for head in range(heads):
            g = head // (heads // kv_heads)
            scores = (cache["k"][:seen, g] @ q[t, head]) * p["scale"]
            weights = torch.softmax(scores, dim=0)
            out[t, head] = weights @ cache["v"][:seen, g]
    return out.reshape(n, heads * dim) @ w["o"].T


def decayed_outer_product_scan(q, k, v, decay, state):
    """Per head: S <- decay_h S + k_t v_t^T, o_t = S^T q_t. q, k: [tokens, heads, dim]; v: [tokens, heads, vdim];
    state [heads, dim, vdim] is updated in place. Returns o [tokens, heads, vdim]."""
    n, heads, _ = q.shape
    out = torch.zeros(n, heads, v.shape[-1], dtype=F64)
    for t in range(n):
        for head in range(heads):
            state[head] = decay[head] * state[head] + torch.outer(k[t, head], v[t, head])
            out[t, head] = state[head].T @ q[t, head]
    return out


def retention(w: dict, p: dict, h: torch.Tensor, state: torch.Tensor, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head, keys scaled by dim^(-1/2), each head's read-out divided by its
    root mean square, gated by silu(W_g h), projected by W_o."""
    n = h.shape[0]
    heads, dim, vdim = p["heads"], p["dim"], p["vdim"]
    q = (h @ w["q"].T).view(n, heads, dim)
    k = (h @ w["k"].T).view(n, heads, dim) * dim ** -0.5
    v = (h @ w["v"].T).view(n, heads, vdim)
    o = decayed_outer_product_scan(q, k, v, torch.tensor(p["decay"], dtype=F64), state)
    o = rms(o, eps).reshape(n, heads * vdim) * silu(h @ w["g"].T)
    return o @ w["o"].T


def parallel_mixer(w: dict, p: dict, h: torch.Tensor, start: int, cache: dict, eps: float) -> torch.Tensor:
    """Softmax attention and retention side by side on the same input: half the sum of the two outputs, each
    RMS-normed over the width with its own weight."""
    if "state" not in cache:
        cache["state"] = torch.zeros(p["right"]["heads"], p["right"]["dim"], p["right"]["vdim"], dtype=F64)
        cache["kv"] = {}
    left = softmax_attention(w["left"], p["left"], h, start, cache["kv"])
    right = retention(w["right"], p["right"], h, cache["state"], eps)
    return 0.5 * (rms(left, eps) * w["left"]["out"] + rms(right, eps) * w["right"]["out"])


def lightning(w: dict, p: dict, h: torch.Tensor, cache: dict, eps: float) -> torch.Tensor:
    """Linear attention on silu-activated q, k, v with a fixed decay per head; all heads RMS-normed together with a
    weight, gated by sigmoid(W_g h), projected by W_o."""
    n = h.shape[0]
    heads, dim, vdim = p["heads"], p["dim"], p["vdim"]
    if "state" not in cache:
        cache["state"] = torch.zeros(heads, dim, vdim, dtype=F64)
    q = silu(h @ w["q"].T).view(n, heads, dim)
    k = silu(h @ w["k"].T).view(n, heads, dim)
    v = silu(h @ w["v"].T).view(n, heads, vdim)
    o = decayed_outer_product_scan(q, k, v, torch.tensor(p["decay"], dtype=F64), cache["state"])
    o = rms(o.reshape(n, heads * vdim), eps) * w["norm"] * sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def short_convolution(x: torch.Tensor, taps: torch.Tensor, history: torch.Tensor):
    """Causal convolution over time per channel. x [tokens, channels]; taps [channels, width], the last column
    multiplying the current token; history [width - 1, channels] holds the inputs before x (zeros at the start).
    Returns (y, new history)."""
    width = taps.shape[1]
    padded = torch.cat([history, x])
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        window = padded[t:t + width]  # inputs t - width + 1 .. t
        y[t] = (window * taps.T).sum(dim=0)
    return y, padded[padded.shape[0] - (width - 1):].clone()


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta(w: dict, p: dict, h: torch.Tensor, cache: dict, eps: float) -> torch.Tensor:
    """The gated delta rule: per head S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    n = h.shape[0]
    heads, kv_heads, dim, vdim, taps = p["heads"], p["kv_heads"], p["dim"], p["vdim"], p["conv"]
    if "state" not in cache:
        cache["state"] = torch.zeros(heads, dim, vdim, dtype=F64)
        for name, channels in (("q", kv_heads * dim), ("k", kv_heads * dim), ("v", heads * vdim)):
            cache["conv_" + name] = torch.zeros(taps - 1, channels, dtype=F64)
    streams = {}
    for name in ("q", "k", "v"):
        y, cache["conv_" + name] = short_convolution(h @ w[name].T, w[name + ".conv"], cache["conv_" + name])
        streams[name] = silu(y)
    q = unit(streams["q"].view(n, kv_heads, dim)) * dim ** -0.5
    k = unit(streams["k"].view(n, kv_heads, dim))
    v = streams["v"].view(n, heads, vdim)
    beta = sigmoid(h @ w["b"].T)
    gate = torch.exp(-torch.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))
    out = torch.zeros(n, heads, vdim, dtype=F64)
    state = cache["state"]
    for t in range(n):
        for head in range(heads):
            j = head // (heads // kv_heads)
            s = gate[t, head] * state[head]
            u = beta[t, head] * (v[t, head] - s.T @ k[t, j])
            s = s + torch.outer(k[t, j], u)
            out[t, head] = s.T @ q[t, j]
            state[head] = s
    out = rms(out, eps) * w["norm"]
    out = out.reshape(n, heads * vdim) * silu(h @ w["g"].T)
    return out @ w["o"].T


def clamped_glu(w: dict, p: dict, h: torch.Tensor) -> torch.Tensor:
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    limit = p["limit"]
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def nested(tensors: dict, prefix: str) -> dict:
    """The tensors under `prefix` as float64, keyed by the rest of their names; "left." and "right." become
    dictionaries of their own."""
    out: dict = {}
    for name, tensor in tensors.items():
        if name.startswith(prefix):
            rest = name[len(prefix):]
            target = out
            if rest.startswith(("left.", "right.")):
                side, rest = rest.split(".", 1)
                target = out.setdefault(side, {})
            target[rest] = tensor.to(F64)
    return out


class PlainTisalorn:
    """The whole model. `forward(tokens, cache)` runs the next tokens of one sequence from `cache` (a dict that starts
    empty) and returns (logits [tokens, vocab], residual stream after every layer run [runs, tokens, width])."""

    def __init__(self, config: dict, tensors: dict) -> None:
        self.config = config
        self.t = {name: value.to(F64) if value.is_floating_point() else value for name, value in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        loop = config.get("loop")
        count = len(config["layers"])
        if loop:
            self.passes = [(t, list(range(loop["start"], loop["stop"]))) for t in range(loop["times"])]
            self.before, self.after = list(range(loop["start"])), list(range(loop["stop"], count))
        else:
            self.passes, self.before, self.after = [], list(range(count)), []

    def layer(self, index: int, x: torch.Tensor, start: int, cache: dict) -> torch.Tensor:
        spec = self.config["layers"][index]
        prefix = f"l{index}."
        h = layer_norm(x, self.t[prefix + "norm1"], self.eps)
        w = nested(self.t, prefix + "mix.")
        if spec["type"] == "parallel":
            x = x + parallel_mixer(w, spec["mixer"], h, start, cache, self.eps)
        elif spec["type"] == "lightning":
            x = x + lightning(w, spec["mixer"], h, cache, self.eps)
        elif spec["type"] == "delta":
            x = x + gated_delta(w, spec["mixer"], h, cache, self.eps)
        else:
            raise ValueError(spec["type"])
        if spec.get("mlp") is not None:
            h = layer_norm(x, self.t[prefix + "norm2"], self.eps)
            x = x + clamped_glu(nested(self.t, prefix + "mlp."), spec["mlp"], h)
        return x

    def forward(self, tokens, cache: dict):
        start = cache.get("length", 0)
        x = self.t["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(self.config["embedding"]["scale"])
        x0 = x
        after_each = []
        run = 0

        def go(indices, x, run):
            for index in indices:
                x = self.layer(index, x, start, cache.setdefault(("run", run), {}))
                after_each.append(x)
                run += 1
            return x, run

        x, run = go(self.before, x, run)
        for t, indices in self.passes:
            x = torch.cat([x, x0], dim=-1) @ self.t["loop.in"].T + self.t["loop.step"][t]
            x, run = go(indices, x, run)
        x, run = go(self.after, x, run)
        cache["length"] = start + len(tokens)
        logits = layer_norm(x, self.t["final.norm"], self.eps) @ self.t["head"].T
        return logits, torch.stack(after_each)
