"""Small Satavik configurations and random weights for the tests: sizes that are no powers of two, one and several
key/value heads, values wider and narrower than the two maps' keys and as wide, part and no rotation, chunks that are no multiple
of a page, layers that borrow another layer's keys, a layer without a feed-forward, one expert of three and three of
five, with and without a shared expert."""
from __future__ import annotations

import math

import torch


def attention(heads=6, kv_heads=2, dim=16, vdim=40, rot_dims=8, base=1e4, scale=0.3, softcap=20.0, diff=0.25, chunk=48,
              kv_from=None, mlp="default"):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
             "diff": diff, "mask": {"size": chunk}, "rot": {"base": base, "dims": rot_dims}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    if mlp == "default":
        mlp = moe()
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def moe(ff=24, limit=0.8, experts=5, top=3, shared_ff=40, shared_limit=1.5):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        out["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return out


def config(layers, vocab=301, width=96, scale=1.7, eps=1e-5) -> dict:
    return {"architecture": "Satavik", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "layers": layers}


CASES = {
    # two layers with keys of their own, two that borrow them crosswise (with other chunks and constants of their
    # own), values wider than both maps' keys together, rotation of half a map
    "borrowed": lambda: config([
        attention(),
        attention(heads=2, kv_heads=1, dim=24, vdim=48, rot_dims=24, base=77.0, chunk=70, diff=0.4, softcap=9.0,
                  mlp=moe(ff=16, experts=3, top=1, shared_ff=0)),
        attention(kv_from=0, chunk=33, scale=0.21, softcap=50.0, diff=0.1, mlp=None),
        attention(heads=4, kv_heads=1, dim=24, vdim=48, rot_dims=24, base=77.0, chunk=1000, kv_from=1, diff=0.4)]),
    # sizes that tile for the tensor cores (maps of 32, values of 64), four query heads per kv head, two kv heads; the
    # second layer borrows with a smaller chunk
    "tiled": lambda: config([
        attention(heads=8, kv_heads=2, dim=32, vdim=64, rot_dims=16, chunk=96, scale=0.18, softcap=15.0,
                  mlp=moe(ff=32, experts=4, top=2, shared_ff=16)),
        attention(heads=8, kv_heads=2, dim=32, vdim=64, rot_dims=16, chunk=40, scale=0.18, softcap=15.0, kv_from=0,
                  mlp=moe(ff=32, experts=4, top=2, shared_ff=16))], width=128, vocab=211),
    # a map size that is no multiple of 8 (no 16-byte pieces), narrow values, no rotation at all, one head, a chunk of
    # five positions, two experts of two
    "narrow": lambda: config([
        attention(heads=1, kv_heads=1, dim=20, vdim=24, rot_dims=0, chunk=5, scale=0.5,
                  mlp=moe(ff=8, experts=2, top=2, shared_ff=8, shared_limit=0.4)),
        attention(heads=3, kv_heads=3, dim=8, vdim=16, rot_dims=2, chunk=64, softcap=3.0)],
        width=64, vocab=97, scale=0.25, eps=3e-4),
}


def random_weights(config_dict: dict, seed: int = 0) -> dict:
    """bfloat16 tensors by checkpoint name, scaled so that activations stay of order one through the layers."""
    g = torch.Generator().manual_seed(seed)
    width = config_dict["width"]
    t: dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        t[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vector(name, size, mean=1.0, spread=0.2):
        t[name] = (mean + spread * torch.randn(size, generator=g)).to(torch.bfloat16)

    matrix("embed", config_dict["vocab"], width, gain=math.sqrt(width))
    matrix("head", config_dict["vocab"], width)
    vector("final.norm", width)
    for i, layer in enumerate(config_dict["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vector(p + "norm1", width)
        matrix(p + "mix.q", m["heads"] * 2 * m["dim"], width, 1.5)
        vector(p + "mix.q.norm", m["dim"], 1.5, 0.4)
        if m.get("kv_from") is None:
            matrix(p + "mix.k", m["kv_heads"] * 2 * m["dim"], width, 1.5)
            matrix(p + "mix.v", m["kv_heads"] * m["vdim"], width, 1.5)
            vector(p + "mix.k.norm", m["dim"], 1.5, 0.4)
        for name in ("lq1", "lk1", "lq2", "lk2"):
            vector(p + "mix." + name, m["dim"], 0.0, 0.6 / math.sqrt(m["dim"]) ** 0.5)
        matrix(p + "mix.g", m["heads"], width, 2.0)
        matrix(p + "mix.o", width, m["heads"] * m["vdim"])
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        vector(p + "norm2", width)
        matrix(p + "mlp.router", mlp["router"]["experts"], width, 4.0)
        vector(p + "mlp.router.b", mlp["router"]["experts"], 0.0, 1.0)
        for e in range(mlp["router"]["experts"]):
            matrix(p + f"mlp.e{e}.gate", mlp["expert"]["ff"], width, 1.5)
            matrix(p + f"mlp.e{e}.up", mlp["expert"]["ff"], width, 1.5)
            matrix(p + f"mlp.e{e}.down", width, mlp["expert"]["ff"])
        if mlp.get("shared") is not None:
            matrix(p + "mlp.shared.gate", mlp["shared"]["ff"], width, 1.5)
            matrix(p + "mlp.shared.up", mlp["shared"]["ff"], width, 1.5)
            matrix(p + "mlp.shared.down", width, mlp["shared"]["ff"])
    return t


def make_engine(config_dict: dict, tensors: dict, dtype: str, max_tokens: int = 2048, **kwargs):
    from etalii.dllm_b200.config.registry import config_from_dict
    from etalii.dllm_b200.engine.engine import Engine

    kwargs.setdefault("max_length", 1024)
    return Engine(config_from_dict(config_dict), tensors, dtype=dtype, device="cuda:0", max_tokens=max_tokens, **kwargs)


def tokens_for(config_dict: dict, lengths, seed: int = 5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, config_dict["vocab"], (n,), generator=g).tolist() for n in lengths]
