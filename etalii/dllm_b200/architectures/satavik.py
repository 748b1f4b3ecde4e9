"""The Satavik design as data: which parts each layer has, the order they run in, and the checkpoint's tensor names.

Every layer norms what its sublayers return, not what they read: x += norm1(mixer(x)); x += norm2(feed_forward(x))
with RMS norms (a layer may have no feed-forward). The mixer is differential attention: two softmax maps per head over
the same values with query and key norms, rotary positions on the first `rot.dims` places of each map (halves),
capped scores, a mask of chunks of `mask.size` positions, the difference normed per head and a sigmoid gate per head.
A layer with `kv_from: j` projects no keys and values: it reads what layer j's cache holds, so the two share one
cache entry. The feed-forward is a mixture of clamped gated experts with a router bias and a shared expert that runs
for every token. Tensor names: `embed`, `head`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.{q,k,v,q.norm,k.norm,lq1,lk1,lq2,lk2,g,o}`, `l<i>.mlp.{router,router.b}`, `l<i>.mlp.e<n>.{gate,up,down}`,
`l<i>.mlp.shared.{gate,up,down}`."""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.satavik import SatavikConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def mixer_spec(width: int, eps: float, m: dict, prefix: str, reader_chunks=None) -> PartSpec:
    shares = m.get("kv_from") is not None
    rot = m.get("rot")
    position = None
    if rot is not None and rot["dims"]:
        position = PartSpec("rotary", {"head_dim": m["dim"], "theta": float(rot["base"]),
                                       "rotary_dim": int(rot["dims"]), "pairing": "halves"})
    mask = m.get("mask")
    params = {"hidden_size": width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "dim": m["dim"],
              "vdim": m["vdim"], "scale": float(m["scale"]), "diff": float(m["diff"]), "eps": eps,
              "softcap": float(m["softcap"]) if m.get("softcap") is not None else 0.0,
              "chunk": int(mask["size"]) if mask is not None else None, "position": position, "shares_keys": shares,
              "reader_chunks": reader_chunks}
    p = prefix + "mix."
    names = {"q": p + "q", "q_norm": p + "q.norm", "g": p + "g", "o": p + "o"}
    names.update({name: p + name for name in ("lq1", "lk1", "lq2", "lk2")})
    if not shares:
        names.update({"k": p + "k", "v": p + "v", "k_norm": p + "k.norm"})
    return PartSpec("differential_attention", params, names)


def feed_forward_spec(width: int, mlp: dict, prefix: str) -> PartSpec:
    p = prefix + "mlp."
    experts = int(mlp["router"]["experts"])
    names = {"router": p + "router", "router_bias": p + "router.b"}
    for e in range(experts):
        names.update({f"e{e}.{part}": f"{p}e{e}.{part}" for part in ("gate", "up", "down")})
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("clamped_glu", {"hidden_size": width, "intermediate_size": int(mlp["shared"]["ff"]),
                                          "limit": float(mlp["shared"]["limit"]), "alpha": 1.702, "shift": 1.0})
        names.update({f"shared.{part}": f"{p}shared.{part}" for part in ("gate", "up", "down")})
    return PartSpec("clamped_glu_experts", {
        "hidden_size": width, "intermediate_size": int(mlp["expert"]["ff"]), "experts": experts,
        "top": int(mlp["router"]["top"]), "limit": float(mlp["expert"]["limit"]), "alpha": 1.702, "shift": 1.0,
        "router_bias": True, "shared": shared}, names)


def build_spec(config: SatavikConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    layers, schedule, entry_of = [], [], {}
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        norm = lambda name: PartSpec("rmsnorm", {"hidden_size": width, "eps": eps}, {"weight": prefix + name})  # noqa: E731
        # a layer's cache entry is read by itself and by the layers that borrow it, each with a mask of its own
        readers = [other["mixer"] for j, other in enumerate(config.layers)
                   if j == index or other["mixer"].get("kv_from") == index]
        sizes = tuple(int(m["mask"]["size"]) if m.get("mask") is not None else None for m in readers)
        mixer = mixer_spec(width, eps, layer["mixer"], prefix, sizes)
        mlp = layer.get("mlp")
        if mlp is None:
            layers.append(LayerSpec(block="output_norm_mixer", parts={"mixer": mixer, "mixer_norm": norm("norm1")}))
        else:
            layers.append(LayerSpec(mixer, feed_forward_spec(width, mlp, prefix), norm("norm1"), norm("norm2"),
                                    block="output_norm"))
        source = layer["mixer"].get("kv_from")
        if source is None:
            entry_of[index] = len(entry_of)  # a cache entry of its own
            schedule.append(ScheduleEntry(index, entry_of[index], True))
        else:
            schedule.append(ScheduleEntry(index, entry_of[source], False))
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=width, max_position=config.max_position,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": width,
                                               "scale": config.embedding_scale}, {"weight": "embed"}),
        layers=tuple(layers),
        final_norm=PartSpec("rmsnorm", {"hidden_size": width, "eps": eps}, {"weight": "final.norm"}),
        head=PartSpec("linear", {"vocab_size": config.vocab, "hidden_size": width}, {"weight": "head"}),
        schedule=tuple(schedule), stop_token_ids=tuple(config.eos_token_ids),
        # (a layer without a feed-forward has no use for a second norm; a checkpoint that stores one all the same loads)
        ignored_suffixes=tuple(f"l{i}.norm2" for i, layer in enumerate(config.layers) if layer.get("mlp") is None),
    )


register_architecture("Satavik", SatavikConfig, build_spec)
