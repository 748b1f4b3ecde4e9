"""Differential attention: every query head has two score maps over the same values, and the head's output is the
first map's weighted sum minus `weight` times the second's.

Per token, from the mixer's input h: q = W_q h [heads x 2 x dim] and k = W_k h [kv_heads x 2 x dim], laid out head by
head as [map 1 | map 2]; v = W_v h [kv_heads x vdim]. Every (head, map) vector of q and k is divided by its root mean
square over `dim` and multiplied by a weight [dim] (one for q, one for k, shared by heads and maps), then its first
`rotary_dim` places turn by the position (pairs i, i + rotary_dim / 2). Scores are q_m . k_m * scale, then
softcap * tanh(score / softcap); a token sees the keys of its own chunk of `chunk` positions up to itself (chunks count
from position 0 of the sequence), and a softmax runs over them, per map. With a1, a2 the two maps' sums over the
same v:

    o = a1 - weight * a2,  weight = exp(lq1 . lk1) - exp(lq2 . lk2) + diff  (one number for the layer)
    o <- o / sqrt(mean(o^2) + eps) * (1 - diff)                               (over the head's vdim values)
    o <- o * sigmoid(W_g h)_head                                              (one gate per head)

and W_o runs over the concatenated heads. Scores, weights, norms, the combination and the gate are float32; the cache
holds keys (both maps, after norm and rotation) and values in the activation type. A mixer built with
`shares_keys=True` has no key, value and key-norm tensors: it reads the cache entry another layer wrote (the schedule
names it) with queries, mask and everything else of its own."""
from __future__ import annotations

import math

import torch

from ..cache.paged import CacheNeed
from ..kernels import ops
from .norm import row_rule
from .registry import build_part, register_part
from .spec import ParamSpec


class DifferentialAttention:
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 diff: float, eps: float, softcap: float = 0.0, chunk: int | None = None, window: int | None = None,
                 position=None, shares_keys: bool = False, reader_chunks=None) -> None:
        """`reader_chunks`: where other mixers read this one's cache entry, the chunk sizes of ALL its readers, this
        one included (None among them: a reader without chunks); the cache keeps a position while any of them can
        still see it. Default: this mixer alone."""
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim = int(dim), int(vdim)
        self.scale, self.diff, self.eps, self.softcap = float(scale), float(diff), float(eps), float(softcap or 0.0)
        self.chunk = int(chunk) if chunk else None
        self.window = int(window) if window else None
        self.shares_keys = bool(shares_keys)
        readers = (self.chunk,) if reader_chunks is None else tuple(reader_chunks)
        self.keep_chunks = None if any(not c for c in readers) else tuple(sorted({int(c) for c in readers}))
        self.position = build_part("position", position) if position is not None else None
        self.w_in = self.w_o = self.q_weight = self.k_weight = None
        self.weight = 0.0

    @staticmethod
    def parameters(hidden_size, num_heads, num_kv_heads, dim, vdim, shares_keys=False, **_) -> dict[str, ParamSpec]:
        heads, kv_heads, dim, vdim = int(num_heads), int(num_kv_heads), int(dim), int(vdim)
        out = {"q": ParamSpec((heads * 2 * dim, hidden_size)), "q_norm": ParamSpec((dim,), "ones")}
        if not shares_keys:
            out.update({"k": ParamSpec((kv_heads * 2 * dim, hidden_size)), "v": ParamSpec((kv_heads * vdim, hidden_size)),
                        "k_norm": ParamSpec((dim,), "ones")})
        out.update({name: ParamSpec((dim,)) for name in ("lq1", "lk1", "lq2", "lk2")})
        out.update({"g": ParamSpec((heads, hidden_size)), "o": ParamSpec((hidden_size, heads * vdim))})
        return out

    def supports(self, rt) -> str | None:
        if self.dim > 256 or self.vdim > 256:
            return f"dim {self.dim}, vdim {self.vdim}: the attention kernel takes at most 256 each"
        return row_rule(rt, hidden_size=self.hidden_size, **{"heads x vdim": self.num_heads * self.vdim})

    def cache_need(self) -> CacheNeed:
        return CacheNeed("kv", kv_heads=self.num_kv_heads, head_dim=2 * self.dim, window=self.window,
                         value_dim=0 if self.vdim == 2 * self.dim else self.vdim, chunk=self.keep_chunks)

    def bind(self, tensors, rt) -> None:
        # one projection for everything a token needs of h: q, then (a mixer with keys of its own) k and v, then the
        # heads' gates
        names = ("q", "g") if self.shares_keys else ("q", "k", "v", "g")
        fused = torch.cat([tensors[name].to(rt.dtype) for name in names], dim=0)
        self.w_in = fused.contiguous().to(rt.device)
        self.w_o = rt.to_device(tensors["o"], rt.dtype)
        self.q_weight = rt.to_device(tensors["q_norm"], torch.float32)
        self.k_weight = None if self.shares_keys else rt.to_device(tensors["k_norm"], torch.float32)
        first = float((tensors["lq1"].float() * tensors["lk1"].float()).sum())
        second = float((tensors["lq2"].float() * tensors["lk2"].float()).sum())
        self.weight = math.exp(first) - math.exp(second) + self.diff
        if self.position is not None:
            self.position.bind({}, rt)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, cache, rt, write_cache: bool = True,
                epilogue: int = ops.EPI_RESIDUAL) -> None:
        """h: the mixer's input [tokens, hidden] in the activation type. Adds the output to `residual` (float32), or
        with `epilogue=ops.EPI_STORE_F32` writes it there."""
        n = batch.n_tokens
        heads, kv_heads, dim, vdim = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        q_size = heads * 2 * dim
        rows = rt.ws.buffer("mixer_rows", (n, self.w_in.shape[0]), torch.float32)
        ops.gemm(rows, h, self.w_in, ops.EPI_STORE_F32)
        writes = write_cache and not self.shares_keys
        k_at = q_size
        v_at = k_at + kv_heads * 2 * dim
        gate_at = q_size if self.shares_keys else v_at + kv_heads * vdim
        table = self.position.table() if self.position is not None else None
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        q = rt.ws.buffer("map_queries", (n, q_size), torch.float32)
        ops.map_prepare(rows, 0, k_at, v_at, q, cache, heads, dim, self.q_weight, self.k_weight, self.eps, table,
                        rotary_dim, batch, writes)
        attended = rt.ws.buffer("attended", (n, heads * vdim), rt.dtype)
        common = (self.scale, self.softcap, self.weight, self.eps, 1.0 - self.diff, self.chunk or 0, self.window or 0,
                  batch)
        if batch.is_decode and ops.diff_attention_decode_supported(cache, heads, dim):
            # single tokens: a block per (token, kv head, stretch of keys) serves the whole group of query heads
            longest = min(batch.max_context, self.chunk or batch.max_context, self.window or batch.max_context)
            splits = ops.diff_attention_decode_splits(n, kv_heads, longest)
            partial = tickets = None
            if splits > 1:
                partial = rt.ws.buffer("map_partial", (n * kv_heads * splits * 2 * (heads // kv_heads) * (vdim + 2),),
                                       torch.float32)
                tickets = rt.ws.zeros("map_tickets", n * kv_heads, torch.int32)
            ops.diff_attention_decode(attended, q, rows, gate_at, cache, heads, dim, *common, splits, partial, tickets)
        elif not batch.is_decode and ops.diff_attention_prefill_supported(cache, dim):
            # portions of prompts: tiles of 64 queries on the tensor cores
            ops.diff_attention_prefill(attended, q, rows, gate_at, cache, heads, dim, *common)
        else:
            ops.diff_attention(attended, q, rows, gate_at, cache, heads, dim, *common)
        ops.gemm(residual, attended, self.w_o, epilogue)

    def kernel_libraries(self, rt) -> set[str]:
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt", "elementwise", "diff_attention"}
        names = {"gemv", "gemv_cluster", "gemm_tcgen05", "elementwise", "diff_attention"}
        if self.dim % 8 == 0 and self.vdim % 8 == 0 and self.dim <= 128 and self.vdim <= 128:
            names |= {"diff_attention_prefill", "diff_attention_decode"}
        return names


register_part("mixer", "differential_attention", DifferentialAttention)
