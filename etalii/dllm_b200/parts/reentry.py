"""Parts that rewrite the residual stream between two runs of the layer schedule (role "reentry"). A model whose
stretch of layers runs several times in a row names one in the schedule entries that begin a round.

"concat_project": x <- W [x | e] + start[round], with e the embedding's output (the stream as it was before the
first layer), W [hidden, 2 hidden] and one start row per round. The product runs in the activation type with float32
sums; the start row is added in float32 (it is what the product's epilogue adds into)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .norm import row_rule
from .registry import register_part
from .spec import ParamSpec


class ConcatProject:
    def __init__(self, hidden_size: int, rounds: int) -> None:
        self.hidden_size, self.rounds = int(hidden_size), int(rounds)
        self.weight = self.starts = None

    @staticmethod
    def parameters(hidden_size, rounds) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((int(hidden_size), 2 * int(hidden_size))),
                "starts": ParamSpec((int(rounds), int(hidden_size)))}

    def supports(self, rt) -> str | None:
        return row_rule(rt, hidden_size=self.hidden_size)

    def bind(self, tensors, rt) -> None:
        self.weight = rt.to_device(tensors["weight"], rt.dtype)
        self.starts = rt.to_device(tensors["starts"], torch.float32)

    def forward(self, x: torch.Tensor, embedded: torch.Tensor, round_index: int, batch, rt) -> None:
        both = rt.ws.buffer("reentry_operand", (batch.n_tokens, 2 * self.hidden_size), rt.dtype)
        ops.concat_restart(both, x, embedded, self.starts[round_index])
        ops.gemm(x, both, self.weight, ops.EPI_RESIDUAL)

    def kernel_libraries(self, rt) -> set[str]:
        return {"elementwise"}


register_part("reentry", "concat_project", ConcatProject)
