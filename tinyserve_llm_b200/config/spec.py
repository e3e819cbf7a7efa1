"""
Architecture-neutral description of a decoder: what the engine builds a model from.

An architecture's typed configuration (for instance `LlamaConfig`) is turned by its registered
builder into a `ModelSpec`: a list of block definitions (each naming a mixer, a feed-forward, its
norms and an arrangement, every size and constant as a field) and a run list that says in which
order the blocks execute and which cache entry each execution uses.  Nothing below this file knows
which architecture it serves.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """Base of every part description. `kind` selects the implementation in the part registry."""

    kind: str = field(init=False, default="")


@dataclass(frozen=True)
class Llama3Scaling:
    """Frequency rescaling of llama3-type rotary embeddings (reference: model/llama.py:107-128)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotate-half rotary position encoding applied to queries and keys."""

    kind: str = field(init=False, default="rotary")
    head_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    scaling: Llama3Scaling | None = None


@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    kind: str = field(init=False, default="rmsnorm")
    size: int = 0
    eps: float = 1e-6


@dataclass(frozen=True)
class StreamRMSNormSpec(PartSpec):
    """
    RMS norm beside a residual stream that is kept in float32 whatever the activation dtype.  The
    weight that multiplies is `weight_offset` + the stored tensor (1.0: a weight stored around zero);
    `weight_name` is the tensor's name behind the part's prefix ("" where the prefix is the name).
    """

    kind: str = field(init=False, default="rmsnorm_stream")
    size: int = 0
    eps: float = 1e-6
    weight_offset: float = 0.0
    weight_name: str = "weight"


@dataclass(frozen=True)
class InlineRotarySpec(PartSpec):
    """
    Rotate-half rotation over the first `dims` channels of a head, channel i paired with i + dims/2,
    angle = position * base^(-2i/dims), computed in float32 inside the kernels (no position table,
    so no longest position).
    """

    kind: str = field(init=False, default="rotary_inline")
    dims: int = 0
    base: float = 10000.0


@dataclass(frozen=True)
class LinearRecurrenceSpec(PartSpec):
    """
    Linear attention as a recurrence over a matrix state per request and head:
    S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; each head's o is RMS-normed over its value
    channels, gated by silu of a projection, and projected out.

    `decay`: "head" (one constant per head, `head_decays`) or "channel_logits" (per key channel,
    a = sigmoid(z)^(1/tau) with z a low-rank projection of the input plus a bias).
    """

    kind: str = field(init=False, default="linear_recurrence")
    hidden_size: int = 0
    num_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    q_scale: float = 1.0                 # multiplies q (after rotation)
    k_scale: float = 1.0                 # multiplies k (after rotation)
    decay: str = "head"
    head_decays: tuple[float, ...] = ()
    decay_rank: int = 0                  # inner size of the low-rank decay projection
    tau: float = 1.0
    position: PartSpec | None = None     # rotation of q and k
    out_norm_weight: bool = True         # the norm of o has a weight (shared by the heads)
    out_norm_eps: float = 1e-6


@dataclass(frozen=True)
class LatentAttentionSpec(PartSpec):
    """
    Softmax attention whose per-head keys and values are up-projections of one cached latent per
    token; queries go through a normed latent of their own; one rotated key part is shared by the heads.
    """

    kind: str = field(init=False, default="latent_attention")
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0                    # unrotated query/key channels a head
    rot_dim: int = 0                     # rotated query/key channels a head
    value_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    window: int = 0                      # 0: every earlier key; w > 0: the last w keys, the query's own included
    norm_eps: float = 1e-6
    position: PartSpec | None = None


@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Causal grouped-query attention over a paged key/value cache."""

    kind: str = field(init=False, default="attention")
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0            # multiplies q.k before the softmax
    window: int = 0               # 0: every earlier key; w > 0: the last w keys, the query's own included
    position: PartSpec | None = None


@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """Dense gated feed-forward: down(act(gate(x)) * up(x))."""

    kind: str = field(init=False, default="gated_mlp")
    hidden_size: int = 0
    intermediate_size: int = 0
    # "silu": silu(g) * u; "relu": relu(g) * u;
    # "clamped_swish": g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit)
    activation: str = "silu"
    limit: float = 0.0
    alpha: float = 1.0
    tensor_names: tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")


@dataclass(frozen=True)
class RoutedExpertsSpec(PartSpec):
    """
    `num_experts` gated feed-forward layers of which each token uses the `top` with the largest router
    logits (float32, with a bias), weighted by the softmax over the chosen logits; an optional shared
    expert runs for every token and is added.  `expert` describes one expert (its tensors live under
    `expert_prefix` with the expert's index in place of "{}").
    """

    kind: str = field(init=False, default="routed_experts")
    hidden_size: int = 0
    num_experts: int = 0
    top: int = 1
    expert: GatedMLPSpec | None = None
    shared: GatedMLPSpec | None = None
    expert_prefix: str = "e{}."
    shared_prefix: str = "shared."
    router_name: str = "router"
    router_bias_name: str | None = "router.b"


@dataclass(frozen=True)
class BlockSpec:
    """
    One layer definition: its parts, how they are wired, and the checkpoint prefix its tensors
    live under.  `arrangement` picks the wiring (the registry of arrangements); "pre_norm" is
    x + mixer(norm(x)) followed by x + ffn(norm(x)) with the adds deferred into the next norm;
    "sandwich_norm" norms each sublayer's output as well, x + norm_b(mixer(norm(x))), around a
    float32 residual stream.
    """

    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec | None    # None (arrangements that allow it): the block has no feed-forward
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec | None
    prefix: str                      # e.g. "model.layers.3."
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."
    # arrangements that also norm each sublayer's output ("sandwich_norm")
    mixer_post_norm: PartSpec | None = None
    feed_forward_post_norm: PartSpec | None = None
    mixer_post_norm_prefix: str = ""
    feed_forward_post_norm_prefix: str = ""


@dataclass(frozen=True)
class RunEntry:
    """
    One execution of a block.  `block` indexes `ModelSpec.blocks` (the same block may be named by
    several entries: shared weights).  `cache_entry` is the cache/state entry this execution uses;
    entries that share a `cache_entry` share keys and values, and only the one with `writes_cache`
    stores into it (the others read what it stored in the same step).
    """

    block: int
    cache_entry: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    blocks: tuple[BlockSpec, ...]
    run: tuple[RunEntry, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_prefix: str
    lm_head_name: str | None         # None: tied to the embedding
    max_positions: int
    eos_token_id: int
    optional_tensors: tuple[str, ...] = ()     # names a checkpoint may carry that the model does not read
    ignored_suffixes: tuple[str, ...] = ()     # tensors whose names end so are skipped (buffers the model recomputes)
    extras: dict[str, Any] = field(default_factory=dict, compare=False)
    embedding_scale: float = 1.0               # multiplies the embedding rows as they start the stream (not the tied head)

    @property
    def num_cache_entries(self) -> int:
        return 1 + max((e.cache_entry for e in self.run), default=-1)
