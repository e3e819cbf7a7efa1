"""
Typed configuration of the Nipizen decoder, read from the keys of its own config.json, and the
`ModelSpec` it turns into.

config.json: `architecture` "Nipizen", `vocab`, `width`, `norm.eps` and `layers`, a list whose entries
give `type` (the mixer: "parallel" or "mlstm"), `mixer` (its sizes and constants) and `mlp` (`kind`
"moe" with `router.experts`, `router.top` and `expert.ff`, or null for a layer without a
feed-forward).  A "parallel" mixer holds `left` (attention: `heads`, `kv_heads`, `dim`, `vdim`,
`scale`, `rot` with `dims`, `base` and an optional `scaling` of `factor`, `original`, `fast`,
`slow`), `right` (gated delta rule: `heads`, `kv_heads`, `dim`, `vdim`, `conv`), `left_scale` and
`right_scale`; an "mlstm" mixer holds `heads`, `dim`, `vdim`, `gate_cap`.  Layers may come in any
order and number; every size is read here and nowhere else.  Tensors: `embed`, `final.norm`, and
per layer `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`.  The inner sizes of the delta
rule's two low-rank projections are the shapes of their tensors (`decay_rank` and `gate_rank`,
optional, are only needed to draw random weights).

What the design fixes stands here as constants: layer norms with a weight and no bias before each
sublayer around a float32 residual stream; the attention has biases on q, k and v, an RMS norm of q
and of k over the whole projection, and a sigmoid output gate; the delta rule makes q and k unit
vectors with 1e-6 under the root and scales q by dim^(-1/2), as the matrix memory scales its q;
experts are up, squared relu, down, chosen by sigmoid scores that multiply the expert's input; the
output head is the embedding table.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from tinyserve_llm_b200.config.duduvik import DEFAULT_MAX_POSITIONS, _get
from tinyserve_llm_b200.config.llama import ConfigError
from tinyserve_llm_b200.config.spec import (
    BlockSpec,
    GatedAttentionSpec,
    GatedDeltaRuleSpec,
    InlineRotarySpec,
    MatrixLSTMSpec,
    ModelSpec,
    ParallelMixerSpec,
    PartSpec,
    PlainMLPSpec,
    RoutedExpertsSpec,
    RunEntry,
    StreamLayerNormSpec,
    YarnScaling,
)

MIXER_TYPES = ("parallel", "mlstm")
UNIT_EPS = 1e-6
DENOMINATOR_EPS = 1e-6


@dataclass(frozen=True)
class NipizenLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None


@dataclass(frozen=True)
class NipizenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[NipizenLayer, ...]
    max_positions: int
    eos_token_id: int
    raw: Mapping[str, Any]

    architecture = "Nipizen"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "NipizenConfig":
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
            if mlp is not None and mlp.get("kind") != "moe":
                raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp.get('kind')!r} is not supported; have ['moe']")
            parsed.append(NipizenLayer(kind, layer["mixer"], mlp))
        eos = raw.get("eos_token_id")
        config = cls(vocab=_get(raw, "vocab", int), width=_get(raw, "width", int), norm_eps=_get(raw, "norm.eps", float),
                     layers=tuple(parsed), max_positions=int(raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
                     eos_token_id=-1 if eos is None else int(eos), raw=raw)
        for i in range(len(parsed)):                       # every size is looked at now, not at the first step
            config.mixer_spec(i), config.feed_forward_spec(i)
        return config

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)

    # ------------------------------------------------------------------ parts of layer i
    @staticmethod
    def _heads(where: str, m: Mapping[str, Any]) -> tuple[int, int]:
        heads, kv_heads = _get(m, "heads", int), _get(m, "kv_heads", int)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads={heads} is not a multiple of kv_heads={kv_heads}")
        return heads, kv_heads

    def _attention(self, where: str, m: Mapping[str, Any]) -> GatedAttentionSpec:
        heads, kv_heads = self._heads(where, m)
        dim = _get(m, "dim", int)
        rot = _get(m, "rot")
        dims, base = _get(rot, "dims", int), _get(rot, "base", float)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims={dims} must be even and at most dim={dim}")
        yarn = None
        if rot.get("scaling"):
            sc = rot["scaling"]
            yarn = YarnScaling(factor=_get(sc, "factor", float), original=_get(sc, "original", float),
                               fast=_get(sc, "fast", float), slow=_get(sc, "slow", float))
            if yarn.factor <= 0 or yarn.original <= 0 or yarn.fast <= 0 or yarn.slow <= 0 or base <= 1:
                raise ConfigError(f"config.json: {where}.rot.scaling needs positive factor, original, fast and slow")
        return GatedAttentionSpec(hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                                  value_dim=_get(m, "vdim", int), scale=_get(m, "scale", float), bias=True, qk_norm=True,
                                  qk_norm_eps=self.norm_eps, output_gate=True,
                                  position=InlineRotarySpec(dims=dims, base=base, yarn=yarn))

    def _delta_rule(self, where: str, m: Mapping[str, Any]) -> GatedDeltaRuleSpec:
        heads, kv_heads = self._heads(where, m)
        dim = _get(m, "dim", int)
        return GatedDeltaRuleSpec(hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, key_dim=dim,
                                  value_dim=_get(m, "vdim", int), conv_taps=_get(m, "conv", int), q_scale=dim ** -0.5,
                                  unit_eps=UNIT_EPS, out_norm_eps=self.norm_eps, decay_rank=int(m.get("decay_rank", 0)),
                                  gate_rank=int(m.get("gate_rank", 0)))

    def mixer_spec(self, i: int) -> PartSpec:
        layer = self.layers[i]
        m, where = layer.mixer, f"layers[{i}].mixer"
        if layer.type == "mlstm":
            dim = _get(m, "dim", int)
            cap = _get(m, "gate_cap", float)
            if cap <= 0:
                raise ConfigError(f"config.json: {where}.gate_cap must be positive, got {cap}")
            return MatrixLSTMSpec(hidden_size=self.width, num_heads=_get(m, "heads", int), key_dim=dim,
                                  value_dim=_get(m, "vdim", int), q_scale=dim ** -0.5, gate_cap=cap,
                                  denominator_eps=DENOMINATOR_EPS, out_norm_eps=self.norm_eps)
        left, right = _get(m, "left"), _get(m, "right")
        return ParallelMixerSpec(branches=(
            (self._attention(where + ".left", left), "left.", _get(m, "left_scale", float)),
            (self._delta_rule(where + ".right", right), "right.", _get(m, "right_scale", float)),
        ))

    def feed_forward_spec(self, i: int) -> PartSpec | None:
        f = self.layers[i].mlp
        if f is None:
            return None
        experts, top = _get(f, "router.experts", int), _get(f, "router.top", int)
        if top > experts:
            raise ConfigError(f"config.json: layers[{i}].mlp.router.top={top} exceeds experts={experts}")
        expert = PlainMLPSpec(hidden_size=self.width, intermediate_size=_get(f, "expert.ff", int), activation="relu2",
                              tensor_names=("up", "down"))
        return RoutedExpertsSpec(hidden_size=self.width, num_experts=experts, top=top, expert=expert, shared=None,
                                 router_bias_name=None, scoring="sigmoid", weight_on="input")


def nipizen_model_spec(config: NipizenConfig) -> ModelSpec:
    """One block per entry of `layers`, each run once in order with a cache entry of its own."""
    norm = StreamLayerNormSpec(size=config.width, eps=config.norm_eps, weight_name="")
    blocks = []
    for i in range(len(config.layers)):
        feed_forward = config.feed_forward_spec(i)
        blocks.append(BlockSpec(
            arrangement="pre_norm_stream",
            mixer=config.mixer_spec(i),
            feed_forward=feed_forward,
            mixer_norm=norm,
            feed_forward_norm=norm if feed_forward is not None else None,
            prefix=f"l{i}.",
            mixer_prefix="mix.",
            feed_forward_prefix="mlp.",
            mixer_norm_prefix="norm1",
            feed_forward_norm_prefix="norm2",
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
    )
