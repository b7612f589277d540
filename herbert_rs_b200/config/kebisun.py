"""The Kebisun decoder's configuration: a list of layers, each with its own mixer and feed-forward.

config.json of this design is nested:

    architecture: "Kebisun"      vocab, width          embedding.scale      norm.eps
    layers: [{type, mixer: {...}, mlp: {...} or null}, ...]
      type "latent_attention": mixer has heads, dim (unrotated), rot_dim (rotated), vdim, q_rank,
            kv_rank, scale, mask.size (window), rot.{base, dims, scaling.{factor, original, fast, slow}}
      type "gla": mixer has heads, dim, vdim, tau
      mlp.kind "dense": ff;   mlp.kind "moe": expert.ff, router.experts, router.top

Every layer is a block whose sublayers read the residual stream itself and whose results pass a
layer norm and a per-channel scale before they join it; the embedding is scaled; the model ends
with a layer norm and a separate output head.  Tensor names: embed, head, final.norm, and per layer
l<i>.{norm1, norm2, ls1, ls2, mix.*, mlp.*}.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from ..errors import ConfigError
from .base import Reader
from .specs import (BlockSpec, GatedLinearAttentionSpec, LatentAttentionSpec, ModelSpec, NormSpec, RoutedFFSpec,
                    ScaledRotarySpec, SwiGLUSpec, identity_schedule)

# No key of the design bounds a sequence's length (angles are computed from the position); the
# cache's own size is the limit.
NO_POSITION_LIMIT = 1 << 30


def _sub(r: Reader, key: str, required: bool = True):
    v = r.raw(key)
    if v is None:
        if required:
            raise ConfigError(f"{r.where}: missing required key '{key}'")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{r.where}: '{key}' must be an object")
    return Reader(v, f"{r.where}.{key}")


@dataclass
class KebisunConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple            # of (mixer spec, feed-forward spec or None)
    source: dict             # the config.json it was read from

    @classmethod
    def from_dict(cls, c: dict) -> "KebisunConfig":
        r = Reader(c)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        emb = _sub(r, "embedding", required=False)
        scale = emb.number("scale", 1.0) if emb is not None else 1.0
        eps = _sub(r, "norm").number("eps")
        if not eps > 0.0:
            raise ConfigError("norm.eps must be > 0")
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            lr = Reader(entry, f"layers[{i}]")
            kind = lr.string("type")
            m = _sub(lr, "mixer")
            if kind == "latent_attention":
                mixer = cls._latent(m, width, eps)
            elif kind == "gla":
                mixer = cls._gla(m, width, eps)
            else:
                raise ConfigError(f"layers[{i}]: unknown layer type {kind!r} (latent_attention, gla)")
            f = _sub(lr, "mlp", required=False)
            layers.append((mixer, cls._ff(f, width) if f is not None else None))
        return cls(vocab, width, float(scale), float(eps), tuple(layers), copy.deepcopy(c))

    @staticmethod
    def _latent(m: Reader, width: int, eps: float) -> LatentAttentionSpec:
        rope_dim = m.integer("rot_dim", minimum=0)
        position = None
        if rope_dim > 0:
            rot = _sub(m, "rot")
            dims = rot.integer("dims", minimum=2)
            if dims != rope_dim or dims % 2:
                raise ConfigError(f"{m.where}: rot.dims ({dims}) must be even and equal rot_dim ({rope_dim})")
            sc = _sub(rot, "scaling", required=False)
            position = ScaledRotarySpec(dims, rot.number("base")) if sc is None else ScaledRotarySpec(
                dims, rot.number("base"), sc.number("factor"), sc.number("original"), sc.number("fast"), sc.number("slow"))
        mask = _sub(m, "mask", required=False)
        return LatentAttentionSpec(
            hidden_size=width, num_heads=m.integer("heads", minimum=1), nope_dim=m.integer("dim", minimum=1),
            rope_dim=rope_dim, v_dim=m.integer("vdim", minimum=1), kv_rank=m.integer("kv_rank", minimum=1),
            scale=m.number("scale"), norm_eps=eps, q_rank=m.integer("q_rank", None, minimum=1), position=position,
            window=mask.integer("size", minimum=1) if mask is not None else None, sink=True, gate=True)

    @staticmethod
    def _gla(m: Reader, width: int, eps: float) -> GatedLinearAttentionSpec:
        tau = m.number("tau")
        if not tau > 0.0:
            raise ConfigError(f"{m.where}: tau must be > 0")
        # the decay's inner size is a tensor's shape, not a key of the design; "decay_rank" is read
        # only so that a configuration can say which size random weights should get
        return GatedLinearAttentionSpec(
            hidden_size=width, num_heads=m.integer("heads", minimum=1), key_dim=m.integer("dim", minimum=1),
            value_dim=m.integer("vdim", minimum=1), decay_rank=m.integer("decay_rank", None, minimum=1),
            decay_tau=tau, norm_eps=eps)

    @staticmethod
    def _ff(f: Reader, width: int):
        kind = f.string("kind")
        if kind == "dense":
            return SwiGLUSpec(width, f.integer("ff", minimum=1), activation="gelu_tanh", names=("gate", "up", "down"))
        if kind == "moe":
            router = _sub(f, "router")
            experts, top = router.integer("experts", minimum=1), router.integer("top", minimum=1)
            if top > experts:
                raise ConfigError(f"{f.where}: router.top ({top}) exceeds router.experts ({experts})")
            return RoutedFFSpec(width, experts, top, _sub(f, "expert").integer("ff", minimum=1), activation="gelu",
                                renormalize=False, router_name="router", expert_names=("e{e}.up", "e{e}.down"))
        raise ConfigError(f"{f.where}: unknown feed-forward kind {kind!r} (dense, moe)")

    def to_dict(self) -> dict:
        return copy.deepcopy(self.source)

    def model_spec(self) -> ModelSpec:
        blocks = []
        for mixer, ff in self.layers:
            blocks.append(BlockSpec(
                mixer=mixer, ffn=ff,
                norm1=NormSpec(self.width, self.norm_eps, kind="layernorm", weight_name="norm1"),
                norm2=NormSpec(self.width, self.norm_eps, kind="layernorm", weight_name="norm2"),
                kind="sublayer_norm", layer_scale=("ls1", "ls2"),
                names=(("norm1", ""), ("mixer", "mix"), ("norm2", ""), ("ffn", "mlp"))))
        return ModelSpec(
            architecture="Kebisun", vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=identity_schedule(len(blocks)),
            final_norm=NormSpec(self.width, self.norm_eps, kind="layernorm", weight_name="norm"),
            tie_word_embeddings=False, max_position=NO_POSITION_LIMIT, stop_token_ids=(),
            layer_prefix="l{i}.", embed_name="embed", final_norm_name="final.norm", head_name="head",
            embedding_scale=self.embedding_scale)
