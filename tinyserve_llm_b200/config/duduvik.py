"""
Typed configuration of the Duduvik decoder, read from the keys of its own config.json, and the
`ModelSpec` it turns into.

config.json: `architecture` "Duduvik", `vocab`, `width`, `embedding.scale`, `norm.eps` and `layers`, a
list whose entries give `type` (the mixer: "gla", "retention" or "latent_attention"), `mixer` (its
sizes and constants) and `mlp` (the feed-forward: `kind` "dense" with `ff`, `kind` "moe" with
`router.experts`, `router.top`, `expert.ff`, `expert.limit` and an optional `shared` expert, or
null for a layer without one).  Layers may come in any order and number; every size is read here
and nowhere else.  Tensors: `embed`, `final.norm`, and per layer `l<i>.norm1`, `l<i>.norm1b`,
`l<i>.norm2`, `l<i>.norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`.  The inner size of gated linear attention's
low-rank decay projection is the shape of its tensors (`mixer.decay_rank`, optional, is only needed
to draw random weights).

What the design fixes stands here as constants: the norms' weights are stored around zero, a layer
norms the input and the output of each sublayer, the residual stream is float32, dense feed-forwards
gate with relu, experts with a clamped swish of slope 1.702, gated linear attention scales q by
dim^(-1/2) and retention scales k by it, and the output head is the embedding table without its scale.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from tinyserve_llm_b200.config.llama import ConfigError
from tinyserve_llm_b200.config.spec import (
    BlockSpec,
    GatedMLPSpec,
    InlineRotarySpec,
    LatentAttentionSpec,
    LinearRecurrenceSpec,
    ModelSpec,
    PartSpec,
    RoutedExpertsSpec,
    RunEntry,
    StreamRMSNormSpec,
)

EXPERT_SWISH_SLOPE = 1.702
MIXER_TYPES = ("gla", "retention", "latent_attention")
DEFAULT_MAX_POSITIONS = 1 << 20       # nothing in the design bounds a sequence; the engine wants a number


def _get(raw: Mapping[str, Any], path: str, kind=None) -> Any:
    node: Any = raw
    for key in path.split("."):
        if not isinstance(node, Mapping) or key not in node:
            raise ConfigError(f"config.json lacks {path!r}")
        node = node[key]
    if kind is int and (isinstance(node, bool) or not isinstance(node, int) or node <= 0):
        raise ConfigError(f"config.json: {path} must be a positive integer, got {node!r}")
    if kind is float:
        if isinstance(node, bool) or not isinstance(node, (int, float)):
            raise ConfigError(f"config.json: {path} must be a number, got {node!r}")
        node = float(node)
    return node


@dataclass(frozen=True)
class DuduvikLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None


@dataclass(frozen=True)
class DuduvikConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple[DuduvikLayer, ...]
    max_positions: int
    eos_token_id: int
    raw: Mapping[str, Any]

    architecture = "Duduvik"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "DuduvikConfig":
        layers = _get(raw, "layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        parsed = []
        for i, layer in enumerate(layers):
            kind = layer.get("type") if isinstance(layer, Mapping) else None
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not supported; have {list(MIXER_TYPES)}")
            if not isinstance(layer.get("mixer"), Mapping):
                raise ConfigError(f"config.json: layers[{i}] lacks its mixer's sizes")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp.get('kind')!r} is not supported; "
                                  "have ['dense', 'moe']")
            parsed.append(DuduvikLayer(kind, layer["mixer"], mlp))
        eos = raw.get("eos_token_id")
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        config = cls(vocab=_get(raw, "vocab", int), width=_get(raw, "width", int),
                     embedding_scale=_get(raw, "embedding.scale", float), norm_eps=_get(raw, "norm.eps", float),
                     layers=tuple(parsed), max_positions=int(max_positions), eos_token_id=-1 if eos is None else int(eos),
                     raw=raw)
        for i in range(len(parsed)):                       # every size is looked at now, not at the first step
            config.mixer_spec(i), config.feed_forward_spec(i)
        return config

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)

    # ------------------------------------------------------------------ parts of layer i
    def _rotary(self, where: str, rot: Mapping[str, Any]) -> InlineRotarySpec:
        dims, base = _get(rot, "dims", int), _get(rot, "base", float)
        if dims % 2:
            raise ConfigError(f"config.json: {where}.rot.dims={dims} must be even")
        return InlineRotarySpec(dims=dims, base=base)

    def mixer_spec(self, i: int) -> PartSpec:
        layer = self.layers[i]
        m, where = layer.mixer, f"layers[{i}].mixer"
        heads, dim, vdim = _get(m, "heads", int), _get(m, "dim", int), _get(m, "vdim", int)
        if layer.type == "gla":
            return LinearRecurrenceSpec(hidden_size=self.width, num_heads=heads, key_dim=dim, value_dim=vdim,
                                        q_scale=dim ** -0.5, k_scale=1.0, decay="channel_logits",
                                        decay_rank=int(m.get("decay_rank", 0)), tau=_get(m, "tau", float),
                                        out_norm_weight=True, out_norm_eps=self.norm_eps)
        if layer.type == "retention":
            decays = tuple(float(d) for d in _get(m, "decay"))
            if len(decays) != heads:
                raise ConfigError(f"config.json: {where}.decay has {len(decays)} entries for {heads} heads")
            rotary = self._rotary(where, _get(m, "rot"))
            if rotary.dims > dim:
                raise ConfigError(f"config.json: {where}.rot.dims={rotary.dims} exceeds dim={dim}")
            return LinearRecurrenceSpec(hidden_size=self.width, num_heads=heads, key_dim=dim, value_dim=vdim,
                                        q_scale=1.0, k_scale=dim ** -0.5, decay="head", head_decays=decays,
                                        position=rotary, out_norm_weight=False, out_norm_eps=self.norm_eps)
        rot_dim = _get(m, "rot_dim", int)
        rotary = self._rotary(where, _get(m, "rot"))
        if rotary.dims != rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims={rotary.dims} differs from rot_dim={rot_dim}")
        mask = m.get("mask")
        window = _get(mask, "size", int) if mask else 0
        return LatentAttentionSpec(hidden_size=self.width, num_heads=heads, head_dim=dim, rot_dim=rot_dim, value_dim=vdim,
                                   q_rank=_get(m, "q_rank", int), kv_rank=_get(m, "kv_rank", int),
                                   scale=_get(m, "scale", float), window=window, norm_eps=self.norm_eps, position=rotary)

    def _expert(self, e: Mapping[str, Any]) -> GatedMLPSpec:
        return GatedMLPSpec(hidden_size=self.width, intermediate_size=_get(e, "ff", int), activation="clamped_swish",
                            limit=_get(e, "limit", float), alpha=EXPERT_SWISH_SLOPE, tensor_names=("gate", "up", "down"))

    def feed_forward_spec(self, i: int) -> PartSpec | None:
        f = self.layers[i].mlp
        if f is None:
            return None
        if f["kind"] == "dense":
            return GatedMLPSpec(hidden_size=self.width, intermediate_size=_get(f, "ff", int), activation="relu",
                                tensor_names=("gate", "up", "down"))
        experts, top = _get(f, "router.experts", int), _get(f, "router.top", int)
        if top > experts:
            raise ConfigError(f"config.json: layers[{i}].mlp.router.top={top} exceeds experts={experts}")
        shared = f.get("shared")
        return RoutedExpertsSpec(hidden_size=self.width, num_experts=experts, top=top, expert=self._expert(_get(f, "expert")),
                                 shared=self._expert(shared) if shared else None)


def duduvik_model_spec(config: DuduvikConfig) -> ModelSpec:
    """One block per entry of `layers`, each run once in order with a cache entry of its own."""
    norm = StreamRMSNormSpec(size=config.width, eps=config.norm_eps, weight_offset=1.0, weight_name="")
    blocks = []
    for i in range(len(config.layers)):
        feed_forward = config.feed_forward_spec(i)
        blocks.append(BlockSpec(
            arrangement="sandwich_norm",
            mixer=config.mixer_spec(i),
            feed_forward=feed_forward,
            mixer_norm=norm,
            feed_forward_norm=norm if feed_forward is not None else None,
            prefix=f"l{i}.",
            mixer_prefix="mix.",
            feed_forward_prefix="mlp.",
            mixer_norm_prefix="norm1",
            feed_forward_norm_prefix="norm2",
            mixer_post_norm=norm,
            feed_forward_post_norm=norm if feed_forward is not None else None,
            mixer_post_norm_prefix="norm1b",
            feed_forward_post_norm_prefix="norm2b",
        ))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        blocks=tuple(blocks),
        run=tuple(RunEntry(block=i, cache_entry=i) for i in range(len(blocks))),
        final_norm=norm,
        embedding_name="embed",
        final_norm_prefix="final.norm",
        lm_head_name=None,
        max_positions=config.max_positions,
        eos_token_id=config.eos_token_id,
        embedding_scale=config.embedding_scale,
    )
