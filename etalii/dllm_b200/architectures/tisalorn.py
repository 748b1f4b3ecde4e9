"""The Tisalorn design as data: which parts each layer has, the order they run in, and the checkpoint's tensor names.

Every layer is pre-norm with layer norms (a weight, no bias): x += mixer(norm1(x)); x += feed_forward(norm2(x)) (a
layer may have no feed-forward). The mixer is one of
  parallel:  softmax attention (grouped queries, rotary positions on interleaved pairs of the first `rot.dims`
             dimensions, the values being the keys before rotation) beside retention (decayed outer products, keys
             times dim^-1/2, read-out normed per head, silu gate); half the sum of the two, each RMS-normed with a weight;
  lightning: decayed outer products on silu-activated q, k, v, read-out normed over all heads with a weight, sigmoid gate;
  delta:     the gated delta rule behind a short causal convolution.
The feed-forward is a gated unit with clamped pre-activations. A stretch of layers may run several times in a row
(`loop`): every run of a layer has a cache entry of its own, and each round begins with x <- W_in [x | embedding
output] + step[round]. Tensor names: `embed`, `head`, `final.norm`, `loop.in`, `loop.step`, and per layer i
`l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`."""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tisalorn import TisalornConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _names(prefix: str, keys) -> dict[str, str]:
    return {key: prefix + key for key in keys}


def _softmax_branch(width: int, m: dict) -> PartSpec:
    position = None
    if m["rot"]["dims"]:
        position = PartSpec("rotary", {"head_dim": m["dim"], "theta": float(m["rot"]["base"]),
                                       "rotary_dim": int(m["rot"]["dims"]), "pairing": "interleaved"})
    return PartSpec("attention", {"hidden_size": width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                                  "head_dim": m["dim"], "scale": float(m["scale"]), "window": None,
                                  "position": position, "values": "keys"})


def _retention_branch(width: int, m: dict, eps: float) -> PartSpec:
    return PartSpec("decay_linear_attention", {
        "hidden_size": width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "decay": tuple(m["decay"]),
        "eps": eps, "input_activation": None, "key_scale": float(m["dim"]) ** -0.5, "norm": "head",
        "norm_weight": False, "gate": "silu"})


def mixer_spec(width: int, eps: float, layer: dict, prefix: str) -> PartSpec:
    m, p = layer["mixer"], prefix + "mix."
    if layer["type"] == "parallel":
        names = {f"left.{k}": f"{p}left.{k}" for k in ("q", "k", "o", "out")}
        names.update({f"right.{k}": f"{p}right.{k}" for k in ("q", "k", "v", "g", "o", "out")})
        return PartSpec("parallel", {"hidden_size": width, "eps": eps, "factor": 0.5,
                                     "left": _softmax_branch(width, m["left"]),
                                     "right": _retention_branch(width, m["right"], eps)}, names)
    if layer["type"] == "lightning":
        return PartSpec("decay_linear_attention", {
            "hidden_size": width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
            "decay": tuple(m["decay"]), "eps": eps, "input_activation": "silu", "key_scale": 1.0, "norm": "all",
            "norm_weight": True, "gate": "sigmoid"}, _names(p, ("q", "k", "v", "g", "o", "norm")))
    names = _names(p, ("q", "k", "v", "g", "b", "a", "A_log", "dt_bias", "norm", "o"))
    names.update({"q_conv": p + "q.conv", "k_conv": p + "k.conv", "v_conv": p + "v.conv"})
    return PartSpec("gated_delta_rule", {"hidden_size": width, "heads": m["heads"], "qk_heads": m["kv_heads"],
                                         "dim": m["dim"], "vdim": m["vdim"], "conv": m["conv"], "eps": eps}, names)


def build_spec(config: TisalornConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        norm = lambda name: PartSpec("layernorm", {"hidden_size": width, "eps": eps}, {"weight": prefix + name})  # noqa: E731
        mixer = mixer_spec(width, eps, layer, prefix)
        mlp = layer.get("mlp")
        if mlp is None:
            layers.append(LayerSpec(block="pre_norm_mixer", parts={"mixer": mixer, "mixer_norm": norm("norm1")}))
            continue
        feed_forward = PartSpec("clamped_glu", {"hidden_size": width, "intermediate_size": mlp["ff"],
                                                "limit": float(mlp["limit"]), "alpha": 1.702, "shift": 1.0},
                                _names(prefix + "mlp.", ("gate", "up", "down")))
        layers.append(LayerSpec(mixer, feed_forward, norm("norm1"), norm("norm2"), block="pre_norm"))

    schedule, reentries = [], ()
    if config.loop is not None:
        start, stop, times = config.loop["start"], config.loop["stop"], config.loop["times"]
        reentries = (PartSpec("concat_project", {"hidden_size": width, "rounds": times},
                              {"weight": "loop.in", "starts": "loop.step"}),)
        runs = [(i, None, 0) for i in range(start)]
        for t in range(times):
            runs += [(i, 0 if i == start else None, t) for i in range(start, stop)]
        runs += [(i, None, 0) for i in range(stop, len(layers))]
        schedule = [ScheduleEntry(layer, cache, True, reentry, t) for cache, (layer, reentry, t) in enumerate(runs)]
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=width, max_position=config.max_position,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": width,
                                               "scale": config.embedding_scale}, {"weight": "embed"}),
        layers=tuple(layers),
        final_norm=PartSpec("layernorm", {"hidden_size": width, "eps": eps}, {"weight": "final.norm"}),
        head=PartSpec("linear", {"vocab_size": config.vocab, "hidden_size": width}, {"weight": "head"}),
        schedule=tuple(schedule), reentries=reentries, stop_token_ids=tuple(config.eos_token_ids),
        # (a layer without a feed-forward has no use for a second norm; a checkpoint that stores one all the same loads)
        ignored_suffixes=tuple(f"l{i}.norm2" for i, layer in enumerate(config.layers) if layer.get("mlp") is None),
    )


register_architecture("Tisalorn", TisalornConfig, build_spec)
