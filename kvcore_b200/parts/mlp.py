"""Gated feed-forward: ``down(silu(gate(x)) * up(x))`` with gate and up in one matrix.

The arithmetic is the reference's (kvcore/model/models/llama3.py:25-45;
kvcore/model/layer/activation.py:8-17).  The packing differs: when the intermediate size is a
multiple of 8, gate and up rows alternate in runs of 8 (gate 0-7, up 0-7, gate 8-15, ...), so that
the decode kernel, whose threads hold rows n and n+8 of a 16-row tile, can apply the activation
in its epilogue; otherwise rows ``[0, I)`` are the gate projection and ``[I, 2I)`` the up projection.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import FEED_FORWARDS, FeedForward, Summed, WeightSlot


# suffixes of a gated feed-forward's tensors behind its name; ``tensor_names`` of a part overrides them
GATED_TENSOR_NAMES = {
    "gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight",
    "gate_bias": "gate_proj.bias", "up_bias": "up_proj.bias", "down_bias": "down_proj.bias",
}


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(
        self,
        *,
        hidden_size: int,
        intermediate_size: int,
        name: str,
        bias: bool = False,
        tensor_names: dict | None = None,
        dtype: torch.dtype,
        device: torch.device,
    ) -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.name = name
        self.tensor_names = dict(GATED_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        inter = self.intermediate_size
        self.group = 8 if inter % 8 == 0 else 0      # run length of the gate/up interleave (0: halves)
        self.gate_up_weight = torch.empty(2 * inter, self.hidden_size, dtype=dtype, device=device)
        self.down_weight = torch.empty(self.hidden_size, inter, dtype=dtype, device=device)
        self.gate_up_bias = torch.empty(2 * inter, dtype=dtype, device=device) if bias else None
        self.down_bias = torch.empty(self.hidden_size, dtype=dtype, device=device) if bias else None

    def _halves(self, packed: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Where the gate and the up tensor go inside a packed ``[2I, ...]`` tensor."""
        inter, group = self.intermediate_size, self.group
        if group == 0:
            return packed[:inter], packed[inter:]
        runs = packed.view(inter // group, 2, group, *packed.shape[1:])
        return runs[:, 0], runs[:, 1]

    def weight_slots(self) -> list[WeightSlot]:
        inter, hidden = self.intermediate_size, self.hidden_size
        gate, up = self._halves(self.gate_up_weight)
        names = {key: f"{self.name}.{suffix}" for key, suffix in self.tensor_names.items()}
        slots = [
            WeightSlot(names["gate"], gate, file_shape=(inter, hidden)),
            WeightSlot(names["up"], up, file_shape=(inter, hidden)),
            WeightSlot(names["down"], self.down_weight),
        ]
        if self.gate_up_bias is not None:
            gate_bias, up_bias = self._halves(self.gate_up_bias)
            slots += [
                WeightSlot(names["gate_bias"], gate_bias, init="normal", file_shape=(inter,)),
                WeightSlot(names["up_bias"], up_bias, init="normal", file_shape=(inter,)),
                WeightSlot(names["down_bias"], self.down_bias, init="normal"),
            ]
        return slots

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        hidden = K.linear_silu_mul(x, self.gate_up_weight, self.gate_up_bias, group=self.group)
        return K.linear(hidden, self.down_weight, self.down_bias)


    def forward_prenorm(self, h, residual, rms_scale, ctx):
        """The layer's norm folded into the gate/up product and the residual sum into the down
        product (decode-sized batches: no kernel of their own for either)."""
        weight, eps = rms_scale
        summed = isinstance(h, Summed)
        hidden, residual = K.norm_linear(None if summed else h, residual, weight, eps, self.gate_up_weight,
                                         self.gate_up_bias, silu_group=self.group,
                                         sumsq=h.sumsq if summed else None)
        pending, sumsq = K.linear_add_residual(hidden, self.down_weight, self.down_bias, residual)
        return (Summed(sumsq) if pending is None else pending), residual


class ClampedGLU(FeedForward):
    """Gated feed-forward with bounded branches: ``g = min(gate(x), limit)``, ``u = clamp(up(x), -limit, limit)``,
    ``down(g * sigmoid(alpha * g) * (u + shift))``.  Gate and up are the two halves of one matrix; no biases."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702,
                 shift: float = 1.0, name: str, tensor_names: dict | None = None,
                 dtype: torch.dtype, device: torch.device) -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        if not self.limit > 0:
            raise ValueError(f"the clamp limit must be positive, got {limit}")
        self.name = name
        self.tensor_names = dict(GATED_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        self.gate_up_weight = torch.empty(2 * self.intermediate_size, self.hidden_size, dtype=dtype, device=device)
        self.down_weight = torch.empty(self.hidden_size, self.intermediate_size, dtype=dtype, device=device)

    def weight_slots(self) -> list[WeightSlot]:
        inter = self.intermediate_size
        return [
            WeightSlot(f"{self.name}.{self.tensor_names['gate']}", self.gate_up_weight[:inter]),
            WeightSlot(f"{self.name}.{self.tensor_names['up']}", self.gate_up_weight[inter:]),
            WeightSlot(f"{self.name}.{self.tensor_names['down']}", self.down_weight),
        ]

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        hidden = K.glu_clamped(K.linear(x, self.gate_up_weight), alpha=self.alpha, limit=self.limit, shift=self.shift)
        return K.linear(hidden, self.down_weight)


FEED_FORWARDS.register("swiglu", SwiGLU)
FEED_FORWARDS.register("clamped_glu", ClampedGLU)

__all__ = ["ClampedGLU", "GATED_TENSOR_NAMES", "SwiGLU"]
