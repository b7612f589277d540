"""The Votapel decoder's configuration: a list of layers, each a parallel block of one attention
mixer and (optionally) a routed feed-forward.

config.json of this design is nested:

    architecture: "Votapel"    vocab, width, max_positions    norm.eps    residual_mult
    layers: [{type, mixer: {...}, mlp: {...} or null}, ...]
      type "attention": mixer has heads, kv_heads, dim (per-head query/key size), vdim (value size;
            the values are the keys, so it equals dim), scale, softcap, q_temp.{coef, every}
      mlp.kind "moe": expert.ff, router.{experts, top, scale, groups.{count, keep}}, shared.ff

Every layer norms the stream once (an RMS norm whose stored weight lies around zero) and adds both
sublayers' results, times one factor, back to it; a learned vector per position joins the embedding;
the model ends with the same kind of norm and a separate output head.  Tensor names: embed, pos,
head, final.norm, and per layer l<i>.{norm1, mix.{q, q.b, k, k.b, sink, o}, mlp.{router,
e<j>.{gate, up, down}, shared.{gate, up, down}}}.

What the design fixes (not keys): the norm's offset of 1, the two largest scores that make a
group's score, sigmoid router scores without renormalisation, silu in the experts.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from ..errors import ConfigError
from .base import Reader
from .specs import AttentionSpec, BlockSpec, ModelSpec, NormSpec, RoutedFFSpec, SwiGLUSpec, identity_schedule

NO_POSITION_LIMIT = 1 << 30
NORM_OFFSET = 1.0       # stored norm weights lie around zero: the factor is 1 + w
GROUP_TOP = 2           # a group's score: the sum of its two largest scores


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
class VotapelConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    residual_mult: float
    layers: tuple            # of (mixer spec, feed-forward spec or None)
    source: dict             # the config.json it was read from

    @classmethod
    def from_dict(cls, c: dict) -> "VotapelConfig":
        r = Reader(c)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        # the position table's length; a configuration without the key leaves it to the stored tensor's shape
        max_positions = r.integer("max_positions", NO_POSITION_LIMIT, minimum=1)
        eps = _sub(r, "norm").number("eps")
        if not eps > 0.0:
            raise ConfigError("norm.eps must be > 0")
        mult = r.number("residual_mult", 1.0)
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            lr = Reader(entry, f"layers[{i}]")
            kind = lr.string("type")
            if kind != "attention":
                raise ConfigError(f"layers[{i}]: unknown layer type {kind!r} (attention)")
            mixer = cls._attention(_sub(lr, "mixer"), width)
            f = _sub(lr, "mlp", required=False)
            layers.append((mixer, cls._ff(f, width) if f is not None else None))
        return cls(vocab, width, max_positions, float(eps), float(mult), tuple(layers), copy.deepcopy(c))

    @staticmethod
    def _attention(m: Reader, width: int) -> AttentionSpec:
        heads = m.integer("heads", minimum=1)
        kv_heads = m.integer("kv_heads", heads, minimum=1)
        if heads % kv_heads:
            raise ConfigError(f"{m.where}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim = m.integer("dim", minimum=1)
        vdim = m.integer("vdim", dim, minimum=1)
        if vdim != dim:
            raise ConfigError(f"{m.where}: the values are the keys, so vdim ({vdim}) must equal dim ({dim})")
        qt = _sub(m, "q_temp", required=False)
        temperature = None
        if qt is not None:
            temperature = (qt.number("coef"), qt.integer("every", minimum=1))
        cap = m.number("softcap", None)
        if cap is not None and not cap > 0.0:
            raise ConfigError(f"{m.where}: softcap must be > 0")
        return AttentionSpec(
            hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, scale=m.number("scale"),
            bias=True, bias_suffix=".b", values_are_keys=True, q_temperature=temperature, softcap=cap, sink=True,
            names=("q", "k", None, "o", "sink"))

    @staticmethod
    def _ff(f: Reader, width: int) -> RoutedFFSpec:
        kind = f.string("kind")
        if kind != "moe":
            raise ConfigError(f"{f.where}: unknown feed-forward kind {kind!r} (moe)")
        router = _sub(f, "router")
        experts, top = router.integer("experts", minimum=1), router.integer("top", minimum=1)
        groups = _sub(router, "groups", required=False)
        count = groups.integer("count", minimum=1) if groups is not None else 1
        keep = groups.integer("keep", minimum=1) if groups is not None else 1
        if experts % count:
            raise ConfigError(f"{f.where}: router.experts ({experts}) is not a multiple of groups.count ({count})")
        if keep > count:
            raise ConfigError(f"{f.where}: groups.keep ({keep}) exceeds groups.count ({count})")
        if top > keep * (experts // count):
            raise ConfigError(f"{f.where}: router.top ({top}) exceeds the {keep * (experts // count)} experts of the kept groups")
        sh = _sub(f, "shared", required=False)
        shared = None
        if sh is not None:
            shared = SwiGLUSpec(width, sh.integer("ff", minimum=1), activation="silu",
                                names=("shared.gate", "shared.up", "shared.down"))
        return RoutedFFSpec(width, experts, top, _sub(f, "expert").integer("ff", minimum=1), activation="silu",
                            renormalize=False, router_name="router", expert_names=("e{e}.gate", "e{e}.up", "e{e}.down"),
                            gated=True, score="sigmoid", groups=count, keep_groups=keep, group_top=GROUP_TOP,
                            weight_scale=router.number("scale", 1.0), shared=shared)

    def to_dict(self) -> dict:
        return copy.deepcopy(self.source)

    def model_spec(self) -> ModelSpec:
        blocks = []
        for mixer, ff in self.layers:
            blocks.append(BlockSpec(
                mixer=mixer, ffn=ff,
                norm1=NormSpec(self.width, self.norm_eps, weight_name="norm1", weight_offset=NORM_OFFSET), norm2=None,
                kind="parallel", residual_mult=self.residual_mult,
                names=(("norm1", ""), ("mixer", "mix"), ("ffn", "mlp"))))
        return ModelSpec(
            architecture="Votapel", vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=identity_schedule(len(blocks)),
            final_norm=NormSpec(self.width, self.norm_eps, weight_name="norm", weight_offset=NORM_OFFSET),
            tie_word_embeddings=False, max_position=self.max_positions, stop_token_ids=(),
            layer_prefix="l{i}.", embed_name="embed", final_norm_name="final.norm", head_name="head",
            position_table_name="pos")
