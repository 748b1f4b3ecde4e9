"""Small Tisalorn configurations and random weights for the tests: sizes that are no powers of two, unequal head
counts, dims that need padding in the kernels, loops of one and several rounds, a layer without a feed-forward."""
from __future__ import annotations

import math

import torch


def parallel(heads=6, kv_heads=2, dim=32, rot_dims=16, base=1e4, scale=0.2, r_heads=3, r_dim=20, r_vdim=8,
             decay=None, ff=136, limit=0.8):
    decay = decay if decay is not None else [1.0 - 2.0 ** -(2 + i) for i in range(r_heads)]
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                               "rot": {"base": base, "dims": rot_dims}, "scale": scale},
                      "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": decay}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def lightning(heads=2, dim=24, vdim=40, decay=None, ff=136, limit=0.8):
    decay = decay if decay is not None else [math.exp(-1.0 / (2 + 30 * i)) for i in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, ff=136, limit=0.8):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def config(layers, loop=None, vocab=301, width=96, scale=1.7, eps=1e-5) -> dict:
    out = {"architecture": "Tisalorn", "vocab": vocab, "width": width, "embedding": {"scale": scale},
           "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CASES = {
    # every mixer, a loop of three rounds from the first layer on, a last layer without a feed-forward
    "mixed": lambda: config([delta(), parallel(), lightning(), delta(heads=2, kv_heads=2, dim=40, vdim=16, conv=2,
                                                                      ff=None)], loop=(0, 2, 3)),
    # no loop; rotation of every dimension of heads of 24 (the general rotation path), one kv head, one decay head
    "plain_order": lambda: config([parallel(heads=4, kv_heads=1, dim=24, rot_dims=24, base=77.0, scale=0.31,
                                            r_heads=1, r_dim=36, r_vdim=56, decay=[0.9]),
                                   lightning(heads=3, dim=8, vdim=8, decay=[1.0, 0.5, 0.0], ff=72, limit=0.3)],
                                  width=64, vocab=97, scale=0.25, eps=3e-4),
    # a loop of ONE round over the last layers; no rotation at all; a convolution of one tap and of five
    "one_round": lambda: config([delta(heads=4, kv_heads=4, dim=12, vdim=12, conv=1),
                                 parallel(heads=2, kv_heads=2, dim=64, rot_dims=0, scale=0.125, r_heads=2, r_dim=64,
                                          r_vdim=64),
                                 delta(heads=6, kv_heads=2, dim=32, vdim=8, conv=5)], loop=(1, 3, 1), width=128),
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
    loop = config_dict.get("loop")
    if loop:
        matrix("loop.in", width, 2 * width, gain=1.4)
        t["loop.step"] = (0.3 * torch.randn(loop["times"], width, generator=g)).to(torch.bfloat16)
    for i, layer in enumerate(config_dict["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vector(p + "norm1", width)
        if layer["type"] == "parallel":
            left, right = m["left"], m["right"]
            matrix(p + "mix.left.q", left["heads"] * left["dim"], width, 2.0)
            matrix(p + "mix.left.k", left["kv_heads"] * left["dim"], width, 2.0)
            matrix(p + "mix.left.o", width, left["heads"] * left["dim"])
            vector(p + "mix.left.out", width)
            for name, rows in (("q", right["heads"] * right["dim"]), ("k", right["heads"] * right["dim"]),
                               ("v", right["heads"] * right["vdim"]), ("g", right["heads"] * right["vdim"])):
                matrix(p + "mix.right." + name, rows, width, 1.5)
            matrix(p + "mix.right.o", width, right["heads"] * right["vdim"])
            vector(p + "mix.right.out", width)
        elif layer["type"] == "lightning":
            for name, rows in (("q", m["heads"] * m["dim"]), ("k", m["heads"] * m["dim"]),
                               ("v", m["heads"] * m["vdim"]), ("g", m["heads"] * m["vdim"])):
                matrix(p + "mix." + name, rows, width, 1.5)
            matrix(p + "mix.o", width, m["heads"] * m["vdim"])
            vector(p + "mix.norm", m["heads"] * m["vdim"])
        else:
            qk, values = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            for name, rows in (("q", qk), ("k", qk), ("v", values), ("g", values), ("b", m["heads"]),
                               ("a", m["heads"])):
                matrix(p + "mix." + name, rows, width, 1.5)
            for name, rows in (("q", qk), ("k", qk), ("v", values)):
                t[p + f"mix.{name}.conv"] = (0.6 * torch.randn(rows, m["conv"], generator=g)).to(torch.bfloat16)
            t[p + "mix.A_log"] = (torch.rand(m["heads"], generator=g) * 2 - 2.5).to(torch.bfloat16)
            t[p + "mix.dt_bias"] = (torch.randn(m["heads"], generator=g)).to(torch.bfloat16)
            vector(p + "mix.norm", m["vdim"])
            matrix(p + "mix.o", width, values)
        if layer.get("mlp") is not None:
            vector(p + "norm2", width)
            matrix(p + "mlp.gate", layer["mlp"]["ff"], width, 1.5)
            matrix(p + "mlp.up", layer["mlp"]["ff"], width, 1.5)
            matrix(p + "mlp.down", width, layer["mlp"]["ff"])
    return t


def make_engine(config_dict: dict, tensors: dict, dtype: str, max_tokens: int = 2048, **kwargs):
    from etalii.dllm_b200.config.registry import config_from_dict
    from etalii.dllm_b200.engine.engine import Engine

    kwargs.setdefault("max_length", 1024)
    return Engine(config_from_dict(config_dict), tensors, dtype=dtype, device="cuda:0", max_tokens=max_tokens, **kwargs)


def tokens_for(config_dict: dict, lengths, seed: int = 5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, config_dict["vocab"], (n,), generator=g).tolist() for n in lengths]
