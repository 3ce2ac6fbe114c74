"""Typed reader of a Toposun model folder's config.json, and its description as parts.

Toposun is a decoder whose layers run their mixer and their feed-forward side by side on a 32-bit
stream, each behind a scale-only layer norm.  Its keys:

    architecture  "Toposun"
    vocab, width  vocabulary and stream width
    norm.eps      eps of every norm of the model
    layers[i]     type ("attention"), mixer {heads, kv_heads, dim, vdim, scale, rot {base, dims},
                  mask {size, keep_first}}, mlp (null | {kind "dense", ff, limit} |
                  {kind "moe", router {experts, top}, expert {ff}, shared {ff} (optional)})

The attention has biased q/k/output projections, no value projection (the values are the keys as
projected), an RMS norm over the whole q and the whole k projection, a rotation of the first
``rot.dims`` entries of each head, and a sliding window of ``mask.size`` positions behind which the
first ``mask.keep_first`` positions stay visible.  The dense feed-forward clamps its branches; the
mixture routes by sigmoid scores, weights the experts' inputs and adds a sigmoid-gated shared expert.
The output head is the embedding table.  Tensors: ``embed``, ``final.norm``, ``l<i>.norm1|norm2``,
``l<i>.mix.{q,k,o}[.b]``, ``l<i>.mix.{q,k}.norm``, ``l<i>.mlp.{gate,up,down}`` or
``l<i>.mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down,sg}}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .config_json import ConfigError
from .model_spec import LayerSpec, ModelSpec, PartSpec, default_schedule

ARCHITECTURE = "Toposun"
# constants the design fixes
DENSE_GATE_SLOPE = 1.702        # g * sigmoid(1.702 g)
DENSE_UP_SHIFT = 1.0            # ... * (u + 1)
DEFAULT_MAX_POSITIONS = 1 << 17  # the design has no position limit; tables are sized from the engine's own


def _need(raw: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(raw, Mapping) or key not in raw:
        raise ConfigError(f"config.json: {where} is missing key {key!r}")
    return raw[key]


def _positive_int(raw: Mapping[str, Any], key: str, where: str, minimum: int = 1) -> int:
    value = _need(raw, key, where)
    if not isinstance(value, int) or isinstance(value, bool) or value < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {value!r}")
    return value


def _number(raw: Mapping[str, Any], key: str, where: str) -> float:
    value = _need(raw, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class ToposunConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[Mapping[str, Any], ...]
    max_positions: int
    stored_dtype: str | None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ToposunConfig":
        layers = _need(raw, "layers", "the model")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        return cls(
            vocab=_positive_int(raw, "vocab", "the model"),
            width=_positive_int(raw, "width", "the model"),
            eps=_number(_need(raw, "norm", "the model"), "eps", "norm"),
            layers=tuple(layers),
            max_positions=int(raw.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)),
            stored_dtype=raw.get("dtype") or raw.get("torch_dtype"),
        )

    # ---- parts ---------------------------------------------------------------------------------
    def _norm(self, tensor: str) -> PartSpec:
        return PartSpec("layernorm", dict(size=self.width, eps=self.eps, name=tensor, tensor=tensor))

    def _mixer(self, index: int, layer: Mapping[str, Any]) -> PartSpec:
        where = f"layers[{index}].mixer"
        kind = _need(layer, "type", f"layers[{index}]")
        if kind != "attention":
            raise ConfigError(f"config.json: layers[{index}].type {kind!r} is not a mixer of this design")
        m = _need(layer, "mixer", f"layers[{index}]")
        heads, kv_heads = _positive_int(m, "heads", where), _positive_int(m, "kv_heads", where)
        dim, vdim = _positive_int(m, "dim", where), _positive_int(m, "vdim", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv_heads}")
        if vdim != dim:
            raise ConfigError(f"config.json: {where}.vdim {vdim} differs from dim {dim}, but the values are the keys")
        rot, mask = _need(m, "rot", where), _need(m, "mask", where)
        rot_dims = _positive_int(rot, "dims", where + ".rot", minimum=0)
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim {dim}, got {rot_dims}")
        position = None
        if rot_dims:
            position = PartSpec("rope", dict(head_dim=dim, rotary_dim=rot_dims, theta=_number(rot, "base", where + ".rot")))
        return PartSpec(
            "paged_attention",
            dict(
                hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                scale=_number(m, "scale", where), bias=True, o_bias=True,
                sliding_window=_positive_int(mask, "size", where + ".mask"),
                keep_first=_positive_int(mask, "keep_first", where + ".mask", minimum=0),
                value_from_key=True, qk_norm="projection", qk_norm_eps=self.eps,
                tensor_names={"q": "q", "k": "k", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "o_bias": "o.b",
                              "q_norm": "q.norm", "k_norm": "k.norm"},
                position=position, name=f"l{index}.mix",
            ),
        )

    def _feed_forward(self, index: int, layer: Mapping[str, Any]) -> PartSpec | None:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        where = f"layers[{index}].mlp"
        name = f"l{index}.mlp"
        plain_names = {"gate": "gate", "up": "up", "down": "down"}
        kind = _need(mlp, "kind", where)
        if kind == "dense":
            return PartSpec("clamped_glu", dict(
                hidden_size=self.width, intermediate_size=_positive_int(mlp, "ff", where),
                limit=_number(mlp, "limit", where), alpha=DENSE_GATE_SLOPE, shift=DENSE_UP_SHIFT,
                tensor_names=plain_names, name=name))
        if kind == "moe":
            router, expert = _need(mlp, "router", where), _need(mlp, "expert", where)
            experts = _positive_int(router, "experts", where + ".router")
            top = _positive_int(router, "top", where + ".router")
            if top > experts:
                raise ConfigError(f"config.json: {where}.router.top {top} exceeds experts {experts}")
            shared = mlp.get("shared")
            shared_spec = None
            if shared is not None:
                shared_spec = PartSpec("swiglu", dict(
                    hidden_size=self.width, intermediate_size=_positive_int(shared, "ff", where + ".shared"),
                    tensor_names=plain_names, name=f"{name}.shared"))
            return PartSpec("routed_experts", dict(
                hidden_size=self.width, num_experts=experts, top_k=top,
                expert_size=_positive_int(expert, "ff", where + ".expert"),
                score="sigmoid", renormalize=False, weight_on="input",
                shared=shared_spec, shared_gate=shared_spec is not None,
                tensor_names={"router": "router", "shared_gate": "shared.sg", "gate": "e{index}.gate",
                              "up": "e{index}.up", "down": "e{index}.down"},
                name=name))
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design")

    def to_model_spec(self) -> ModelSpec:
        layers = []
        for index, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{index}] is not an object")
            feed_forward = self._feed_forward(index, layer)
            norms = {"mixer_norm": self._norm(f"l{index}.norm1")}
            if feed_forward is not None:
                norms["feed_forward_norm"] = self._norm(f"l{index}.norm2")
            layers.append(LayerSpec(
                prefix=f"l{index}", block=PartSpec("parallel_residual"), mixer=self._mixer(index, layer),
                feed_forward=feed_forward, norms=norms))
        return ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab,
            hidden_size=self.width,
            layers=tuple(layers),
            schedule=default_schedule(len(layers)),
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=self.width,
                                                       name="embed", tensor="embed")),
            final_norm=self._norm("final.norm"),
            lm_head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=self.width, name="lm_head",
                                             tied_to="embed")),
            max_position_embeddings=self.max_positions,
            stored_dtype=self.stored_dtype,
        )


__all__ = ["ARCHITECTURE", "ToposunConfig"]
