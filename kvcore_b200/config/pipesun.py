"""Typed reader of a Pipesun model folder's config.json, and its description as parts.

Pipesun is a decoder on a 32-bit stream whose layers put an RMS norm in front of and behind each
sub-layer, shift the mixer's input towards the token in front, and hand on a learned weighted average of
the results of all layers so far.  Its keys:

    architecture  "Pipesun"
    vocab, width  vocabulary and stream width
    norm.eps      eps of every norm of the model
    layers[i]     type ("attention" | "latent_attention"), mixer {...}, mlp (null | {kind "dense", ff})
      attention         mixer {heads, kv_heads, dim, vdim, scale, diff, kv_from (optional)}: two score maps
                        a head over shared values, per-vector RMS norm of q and k, biased q/k/v projections,
                        no position encoding; ``kv_from: j`` reads layer j's cached keys and values
      latent_attention  mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}}: one cached
                        latent vector a token, interleaved rotary pairs on the rot_dim part, a sink per
                        head, a sigmoid output gate

Tensors: ``embed``, ``head``, ``final.norm``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.shift``,
``l<i>.dwa``, ``l<i>.mix.*`` (see ``parts/attention_maps.py``), ``l<i>.mlp.{gate,up,down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .config_json import ConfigError
from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Pipesun"
DEFAULT_MAX_POSITIONS = 1 << 17   # the design has no position limit of its own


def _need(raw: Any, key: str, where: str) -> Any:
    if not isinstance(raw, Mapping) or key not in raw:
        raise ConfigError(f"config.json: {where} is missing key {key!r}")
    return raw[key]


def _int(raw: Any, key: str, where: str, minimum: int = 1) -> int:
    value = _need(raw, key, where)
    if not isinstance(value, int) or isinstance(value, bool) or value < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {value!r}")
    return value


def _number(raw: Any, key: str, where: str) -> float:
    value = _need(raw, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class PipesunConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[Mapping[str, Any], ...]
    max_positions: int
    stored_dtype: str | None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "PipesunConfig":
        layers = _need(raw, "layers", "the model")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        for index, layer in enumerate(layers):
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{index}] is not an object")
        return cls(
            vocab=_int(raw, "vocab", "the model"),
            width=_int(raw, "width", "the model"),
            eps=_number(_need(raw, "norm", "the model"), "eps", "norm"),
            layers=tuple(layers),
            max_positions=int(raw.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)),
            stored_dtype=raw.get("dtype") or raw.get("torch_dtype"),
        )

    # ---- parts ---------------------------------------------------------------------------------
    def _norm(self, tensor: str) -> PartSpec:
        return PartSpec("rmsnorm_stream", dict(size=self.width, eps=self.eps, name=tensor, tensor=tensor))

    def _attention(self, index: int, m: Mapping[str, Any]) -> tuple[PartSpec, int | None]:
        where = f"layers[{index}].mixer"
        heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv_heads}")
        rot = m.get("rot")
        if isinstance(rot, Mapping) and rot.get("dims"):
            raise ConfigError(f"config.json: {where}.rot: positions do not enter the scores of this mixer")
        source = m.get("kv_from")
        if source is not None:
            if not isinstance(source, int) or isinstance(source, bool) or not 0 <= source < index:
                raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer, got {source!r}")
            other = self.layers[source]
            theirs = other.get("mixer") if isinstance(other.get("mixer"), Mapping) else {}
            if other.get("type") != "attention" or theirs.get("kv_from") is not None:
                raise ConfigError(f"config.json: {where}.kv_from {source} names a layer without keys and values of its own")
            for key in ("kv_heads", "dim", "vdim"):
                if theirs.get(key) != m.get(key):
                    raise ConfigError(f"config.json: {where}.{key} differs from layer {source}'s, whose keys and values it reads")
        spec = PartSpec("differential_attention", dict(
            hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=_int(m, "dim", where),
            value_dim=_int(m, "vdim", where), scale=_number(m, "scale", where), diff=_number(m, "diff", where),
            eps=self.eps, own_kv=source is None, name=f"l{index}.mix"))
        return spec, source

    def _latent_attention(self, index: int, m: Mapping[str, Any]) -> PartSpec:
        where = f"layers[{index}].mixer"
        rot = _need(m, "rot", where)
        rot_dim = _int(m, "rot_dim", where, minimum=0)
        dims = _int(rot, "dims", where + ".rot", minimum=0)
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most rot_dim {rot_dim}, got {dims}")
        return PartSpec("latent_attention", dict(
            hidden_size=self.width, num_heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
            rot_dim=rot_dim, value_dim=_int(m, "vdim", where), kv_rank=_int(m, "kv_rank", where),
            scale=_number(m, "scale", where), eps=self.eps, rot_base=_number(rot, "base", where + ".rot"),
            rot_dims=dims, name=f"l{index}.mix"))

    def _feed_forward(self, index: int, layer: Mapping[str, Any]) -> PartSpec | None:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        where = f"layers[{index}].mlp"
        kind = _need(mlp, "kind", where)
        if kind != "dense":
            raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design")
        return PartSpec("swiglu", dict(
            hidden_size=self.width, intermediate_size=_int(mlp, "ff", where),
            tensor_names={"gate": "gate", "up": "up", "down": "down"}, name=f"l{index}.mlp"))

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        count = len(self.layers)
        for index, layer in enumerate(self.layers):
            kind = _need(layer, "type", f"layers[{index}]")
            mixer_keys = _need(layer, "mixer", f"layers[{index}]")
            source = None
            if kind == "attention":
                mixer, source = self._attention(index, mixer_keys)
            elif kind == "latent_attention":
                mixer = self._latent_attention(index, mixer_keys)
            else:
                raise ConfigError(f"config.json: layers[{index}].type {kind!r} is not a mixer of this design")
            feed_forward = self._feed_forward(index, layer)
            prefix = f"l{index}"
            norms = {"mixer_norm": self._norm(f"{prefix}.norm1"), "mixer_out_norm": self._norm(f"{prefix}.norm1b")}
            if feed_forward is not None:
                norms["feed_forward_norm"] = self._norm(f"{prefix}.norm2")
                norms["feed_forward_out_norm"] = self._norm(f"{prefix}.norm2b")
            # layer i averages the embedded tokens and the results of layers 0..i: i + 1 results in front of
            # its own, count + 1 in the model
            block = PartSpec("sandwich_residual", dict(
                hidden_size=self.width, token_shift=f"{prefix}.shift", depth_average=f"{prefix}.dwa",
                depth=index + 1, depth_slots=count + 1))
            layers.append(LayerSpec(prefix=prefix, block=block, mixer=mixer, feed_forward=feed_forward, norms=norms))
            schedule.append(ScheduleEntry(layer=index, cache_of=source))
        return ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab,
            hidden_size=self.width,
            layers=tuple(layers),
            schedule=tuple(schedule),
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=self.width,
                                                       name="embed", tensor="embed")),
            final_norm=self._norm("final.norm"),
            lm_head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=self.width, name="head",
                                             tensor="head")),
            max_position_embeddings=self.max_positions,
            stored_dtype=self.stored_dtype,
        )


__all__ = ["ARCHITECTURE", "PipesunConfig"]
