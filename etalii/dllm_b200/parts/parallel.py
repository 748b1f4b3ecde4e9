"""Two mixers side by side on the same input: out = factor * (rms(left(h)) * w_left + rms(right(h)) * w_right), each
branch's output divided by its root mean square over the model width and multiplied by a weight of its own before
the sum goes into the residual stream (float32). Either branch is any registered mixer that can write its output to a
buffer instead of adding it to the stream (`forward(..., epilogue=ops.EPI_STORE_F32)`); each keeps its own cache
entry (keys and values, a state, or several)."""
from __future__ import annotations

import torch

from ..cache.paged import CacheNeed
from ..kernels import ops
from .registry import build_part, part_factory, register_part
from .spec import ParamSpec, PartSpec

_SIDES = ("left", "right")


class ParallelMixer:
    def __init__(self, hidden_size: int, eps: float, left: PartSpec, right: PartSpec, factor: float = 0.5) -> None:
        self.hidden_size, self.eps, self.factor = int(hidden_size), float(eps), float(factor)
        self.branches = [build_part("mixer", left), build_part("mixer", right)]
        self.weights: list = [None, None]
        needs = [b.cache_need() if hasattr(b, "cache_need") else None for b in self.branches]
        self._needs = needs

    @staticmethod
    def parameters(hidden_size, left, right, **_) -> dict[str, ParamSpec]:
        out = {}
        for side, spec in zip(_SIDES, (left, right)):
            declared = part_factory("mixer", spec.kind).parameters(**dict(spec.params))
            out.update({f"{side}.{name}": param for name, param in declared.items()})
            out[f"{side}.out"] = ParamSpec((int(hidden_size),), "ones")
        return out

    def supports(self, rt) -> str | None:
        for side, branch in zip(_SIDES, self.branches):
            reason = branch.supports(rt) if hasattr(branch, "supports") else None
            if reason:
                return f"{side}: {reason}"
        return None

    def cache_need(self) -> CacheNeed | None:
        present = [need for need in self._needs if need is not None]
        if not present:
            return None
        return CacheNeed("several", parts=tuple(present))

    def bind(self, tensors, rt) -> None:
        for index, (side, branch) in enumerate(zip(_SIDES, self.branches)):
            prefix = side + "."
            own = {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}
            self.weights[index] = rt.to_device(own.pop("out"), torch.float32)
            branch.bind(own, rt)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, cache, rt, write_cache: bool = True) -> None:
        views = iter(cache if isinstance(cache, (tuple, list)) else (cache,))
        outputs = []
        for index, (branch, need) in enumerate(zip(self.branches, self._needs)):
            out = rt.ws.buffer(f"branch_{index}", (batch.n_tokens, self.hidden_size), torch.float32)
            branch.forward(h, out, batch, next(views) if need is not None else None, rt, write_cache,
                           epilogue=ops.EPI_STORE_F32)
            outputs.append(out)
        ops.norm_sum_residual(residual, outputs[0], self.weights[0], outputs[1], self.weights[1], self.eps,
                              self.factor)

    def kernel_libraries(self, rt) -> set[str]:
        names = {"elementwise"}
        for branch in self.branches:
            if hasattr(branch, "kernel_libraries"):
                names |= set(branch.kernel_libraries(rt))
        return names


register_part("mixer", "parallel", ParallelMixer)
