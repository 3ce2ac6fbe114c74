"""Grouped-query attention over the paged cache.

Order of operations as in the reference's attention layer
(kvcore/model/models/llama3.py:87-104; kvcore/model/layer/attention.py:53-96;
kvcore/model/attn_backend/torch_paged.py:90-117, 151-166): one packed q/k/v projection,
position encoding on q and k, keys and values of this step's tokens written into their
pages, then every query attends over its request's cached positions up to its own
(optionally only the trailing ``sliding_window`` of them) with 32-bit scores, softmax and
accumulation, and the output projection.  Query head ``h`` reads kv head ``h // (H/KVH)``.

Variants, each a constructor parameter: ``keep_first`` first positions that stay visible behind the
sliding window; ``value_from_key`` (no value projection: the values are the keys as projected, before
any norm or rotation); ``qk_norm`` (an RMS norm of q and of k ahead of the rotation, over the whole
projection or per head); a position encoding that turns only part of each head; ``tensor_names`` for
checkpoints that name the projections differently.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..config.model_spec import PartSpec
from .base import MIXERS, POSITION_ENCODINGS, CacheSpec, Mixer, Summed, WeightSlot


class PagedAttention(Mixer):
    @property
    def graph_safe(self) -> bool:
        return self.position is None or self.position.graph_safe

    def __init__(
        self,
        *,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        scale: float,
        name: str,
        bias: bool = False,
        sliding_window: int | None = None,
        keep_first: int = 0,
        value_from_key: bool = False,
        qk_norm: str | None = None,
        qk_norm_eps: float = 1e-6,
        o_bias: bool | None = None,
        tensor_names: dict | None = None,
        position: PartSpec | None = None,
        dtype: torch.dtype,
        device: torch.device,
    ) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} must be a multiple of num_kv_heads {num_kv_heads}")
        if sliding_window is not None and sliding_window <= 0:
            raise ValueError(f"sliding_window must be positive when set, got {sliding_window}")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.scale = float(scale)
        self.sliding_window = None if sliding_window is None else int(sliding_window)
        self.keep_first = int(keep_first)
        if self.keep_first < 0 or (self.keep_first and self.sliding_window is None):
            raise ValueError(f"keep_first must be >= 0 and needs a sliding window, got {keep_first}")
        self.value_from_key = bool(value_from_key)
        if qk_norm not in (None, "projection", "head"):
            raise ValueError(f"qk_norm must be None, 'projection' or 'head', got {qk_norm!r}")
        self.qk_norm = qk_norm
        self.qk_norm_eps = float(qk_norm_eps)
        self.tensor_names = dict(self.DEFAULT_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        self.name = name
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        K.check_attention_shape(self.num_heads, self.num_kv_heads, self.head_dim, dtype)
        # the projections are one packed matrix: q rows, k rows, and v rows unless the values are the keys
        packed = self.q_size + (1 if self.value_from_key else 2) * self.kv_size
        self.qkv_weight = torch.empty(packed, self.hidden_size, dtype=dtype, device=device)
        self.o_weight = torch.empty(self.hidden_size, self.q_size, dtype=dtype, device=device)
        self.qkv_bias = torch.empty(packed, dtype=dtype, device=device) if bias else None
        o_bias = bias if o_bias is None else o_bias
        self.o_bias = torch.empty(self.hidden_size, dtype=dtype, device=device) if o_bias else None
        self.q_norm_weight = self.k_norm_weight = None
        if qk_norm is not None:
            q_len, k_len = (self.q_size, self.kv_size) if qk_norm == "projection" else (self.head_dim,) * 2
            self.q_norm_weight = torch.empty(q_len, dtype=dtype, device=device)
            self.k_norm_weight = torch.empty(k_len, dtype=dtype, device=device)
        self.position = (
            None
            if position is None
            else POSITION_ENCODINGS.build(position, dtype=dtype, device=device)
        )

    DEFAULT_TENSOR_NAMES = {
        "q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
        "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias",
        "q_norm": "q_norm.weight", "k_norm": "k_norm.weight",
    }

    def cache_spec(self) -> CacheSpec:
        return CacheSpec.keys_and_values(self.num_kv_heads, self.head_dim, self.sliding_window, self.keep_first)

    def _tensor(self, key: str) -> str:
        return f"{self.name}.{self.tensor_names[key]}"

    def weight_slots(self) -> list[WeightSlot]:
        q, kv = self.q_size, self.kv_size
        slots = [
            WeightSlot(self._tensor("q"), self.qkv_weight[:q]),
            WeightSlot(self._tensor("k"), self.qkv_weight[q : q + kv]),
            WeightSlot(self._tensor("o"), self.o_weight),
        ]
        if not self.value_from_key:
            slots.append(WeightSlot(self._tensor("v"), self.qkv_weight[q + kv :]))
        if self.qkv_bias is not None:
            slots += [
                WeightSlot(self._tensor("q_bias"), self.qkv_bias[:q], init="normal"),
                WeightSlot(self._tensor("k_bias"), self.qkv_bias[q : q + kv], init="normal"),
            ]
            if not self.value_from_key:
                slots.append(WeightSlot(self._tensor("v_bias"), self.qkv_bias[q + kv :], init="normal"))
        if self.o_bias is not None:
            slots.append(WeightSlot(self._tensor("o_bias"), self.o_bias, init="normal"))
        if self.qk_norm is not None:
            slots += [
                WeightSlot(self._tensor("q_norm"), self.q_norm_weight, init="ones"),
                WeightSlot(self._tensor("k_norm"), self.k_norm_weight, init="ones"),
            ]
        if self.position is not None:
            slots += self.position.weight_slots()
        return slots

    def ignorable_tensor_names(self) -> list[str]:
        return [] if self.position is None else self.position.ignorable_tensor_names()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        out = self._attend(K.linear(x, self.qkv_weight, self.qkv_bias), ctx, cache)
        return K.linear(out, self.o_weight, self.o_bias)

    def forward_prenorm(self, h, residual, rms_scale, ctx, cache):
        """The layer's norm folded into the q/k/v product and the residual sum into the output
        product (decode-sized batches: no kernel of their own for either)."""
        weight, eps = rms_scale
        summed = isinstance(h, Summed)
        qkv, residual = K.norm_linear(None if summed else h, residual, weight, eps, self.qkv_weight, self.qkv_bias,
                                      sumsq=h.sumsq if summed else None)
        out = self._attend(qkv, ctx, cache)
        pending, sumsq = K.linear_add_residual(out, self.o_weight, self.o_bias, residual)
        return (Summed(sumsq) if pending is None else pending), residual

    def _needs_preparation(self) -> bool:
        """Whether what lies between the projection and the attention is more than a rotation of whole
        heads: then one kernel does norm, rotation and cache write, and the attention kernels read q and
        the cache as they are."""
        partial = self.position is not None and getattr(self.position, "rotary_dim", self.head_dim) != self.head_dim
        return self.value_from_key or self.qk_norm is not None or partial

    def _attend(self, qkv: torch.Tensor, ctx, cache) -> torch.Tensor:
        table = ctx.block_table(cache.group)
        if self._needs_preparation():
            cos_sin = None if self.position is None else self.position.cos_sin(ctx)
            if cos_sin is None and self.position is not None:
                raise NotImplementedError("attention with a q/k norm or keys as values needs a position "
                                          "encoding that offers its cos/sin table")
            K.qk_prepare(
                qkv, ctx.positions, ctx.req_index, cos_sin, table, cache.k, cache.v,
                self.num_heads, self.num_kv_heads, self.head_dim,
                rotary_dim=None if self.position is None else self.position.rotary_dim,
                norm=self.qk_norm, q_norm_weight=self.q_norm_weight, k_norm_weight=self.k_norm_weight,
                eps=self.qk_norm_eps, value_from_key=self.value_from_key, write_kv=cache.owner,
            )
            return K.paged_attention(
                qkv, cache.k, cache.v, table, ctx,
                self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.sliding_window,
                keep_first=self.keep_first,
            )
        # an encoding that offers its angles as a table gets its rotation fused with the cache write
        cos_sin = None if self.position is None else self.position.cos_sin(ctx)
        if cos_sin is None and self.position is not None:
            tokens = qkv.shape[0]
            q = qkv[:, : self.q_size].view(tokens, self.num_heads, self.head_dim)
            k = qkv[:, self.q_size : self.q_size + self.kv_size].view(
                tokens, self.num_kv_heads, self.head_dim
            )
            self.position.apply(q, k if cache.owner else None, ctx)
        # rotation and cache write run inside the decode kernel where that one is taken, in a
        # kernel in front of the attention otherwise
        return K.paged_attention(
            qkv, cache.k, cache.v, table, ctx,
            self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.sliding_window,
            cos_sin=cos_sin, write_kv=cache.owner, keep_first=self.keep_first,
        )


MIXERS.register("paged_attention", PagedAttention)

__all__ = ["PagedAttention"]
