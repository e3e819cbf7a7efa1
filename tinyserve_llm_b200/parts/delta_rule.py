"""
Gated delta rule: a matrix state per request and value head that is decayed, corrected towards the
current value along the current key, and read with the query.

    q, k, v = silu(short_conv(W h))        causal convolution over time per channel, its last inputs carried
    q, k    <- unit vectors per head (x / sqrt(sum x^2 + unit_eps)),  q <- q * q_scale
    beta = sigmoid(W_b h)                   a = exp(-exp(A_log) softplus(W_a2 (W_a1 h) + dt_bias))
    S <- diag(a) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q       per value head, S [key_dim, value_dim]
    y = W_o ( o / rms(o) * w * sigmoid(W_g2 (W_g1 h)) )

Value head h uses q/k head h // (heads / kv_heads).  The state (float32: the matrices, then the
convolution's last taps - 1 inputs) lives in the request's slot of the cache manager, so prompts in
portions, decoding and mixed batches are one code path.  Beta's projection and the decay logits
leave their products in float32; everything from the convolution's output on is float32.

Like `GatedAttention` the mixer stands alone or inside a `ParallelMixer` (`input_rows`, `inner`,
`out_weight`).
"""

from __future__ import annotations

import dataclasses

import torch

from tinyserve_llm_b200.config.spec import GatedDeltaRuleSpec
from tinyserve_llm_b200.parts.base import Mixer, Runtime, TensorDecl, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows

MAX_KEY_DIM = 256       # csrc/linear_recurrence.cu


@register_part("mixer", "gated_delta_rule")
class GatedDeltaRule(Mixer):
    graph_safe = True

    @classmethod
    def validate(cls, spec: GatedDeltaRuleSpec) -> None:
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"num_heads={spec.num_heads} is not a multiple of num_kv_heads={spec.num_kv_heads}")
        if not 0 < spec.key_dim <= MAX_KEY_DIM:
            raise ValueError(f"key_dim={spec.key_dim} is not supported: the recurrence kernel takes up to {MAX_KEY_DIM}")
        if spec.conv_taps < 1:
            raise ValueError(f"conv_taps={spec.conv_taps}: the convolution has at least the current token's tap")

    @classmethod
    def declare(cls, spec: GatedDeltaRuleSpec) -> dict[str, TensorDecl]:
        cls.validate(spec)
        qk, vv, hidden, taps = spec.num_kv_heads * spec.key_dim, spec.num_heads * spec.value_dim, spec.hidden_size, spec.conv_taps
        ra = spec.decay_rank if spec.decay_rank > 0 else -1          # -1: the checkpoint's own size
        rg = spec.gate_rank if spec.gate_rank > 0 else -1
        return {
            "q": TensorDecl((qk, hidden)), "q.conv": TensorDecl((qk, taps)),
            "k": TensorDecl((qk, hidden)), "k.conv": TensorDecl((qk, taps)),
            "v": TensorDecl((vv, hidden)), "v.conv": TensorDecl((vv, taps)),
            "b": TensorDecl((spec.num_heads, hidden)), "A_log": TensorDecl((spec.num_heads,)),
            "norm": TensorDecl((spec.value_dim,), init="unit"),
            "a1": TensorDecl((ra, hidden)), "a2": TensorDecl((spec.num_heads * spec.key_dim, ra)),
            "dt_bias": TensorDecl((spec.num_heads * spec.key_dim,)),
            "g1": TensorDecl((rg, hidden)), "g2": TensorDecl((vv, rg)),
            "o": TensorDecl((hidden, vv)),
        }

    def __init__(self, spec: GatedDeltaRuleSpec, tensors: dict[str, torch.Tensor], rt: Runtime, fused: bool = False) -> None:
        super().__init__(spec, tensors, rt)
        self.validate(spec)
        for a, b in (("a1", "a2"), ("g1", "g2")):
            if tensors[a].shape[0] != tensors[b].shape[1]:
                raise ValueError(f"the inner sizes of {a} and {b} differ: {tuple(tensors[a].shape)} and {tuple(tensors[b].shape)}")
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.decay_rank, self.gate_rank = int(tensors["a1"].shape[0]), int(tensors["g1"].shape[0])
        self.channels = 2 * spec.num_kv_heads * spec.key_dim + spec.num_heads * spec.value_dim
        # one projection for what reads h and may be rounded: columns [q | k | v | a1 h | g1 h]
        self.input_rows = fuse_rows([tensors["q"], tensors["k"], tensors["v"], tensors["a1"], tensors["g1"]])
        self.out_weight = tensors["o"]
        self.inner_width = spec.num_heads * spec.value_dim
        self.taps = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0).to(**f32).contiguous()
        self.beta = Linear(tensors["b"], rt)
        self.decay_up = Linear(tensors["a2"], rt)
        self.gate_up = Linear(tensors["g2"], rt)
        self.dt_bias = tensors["dt_bias"].to(**f32).contiguous()
        self.a_log = tensors["A_log"].to(**f32).contiguous()
        self.norm_weight = tensors["norm"].to(**f32).contiguous()
        self.matrix_bytes = spec.num_heads * spec.key_dim * spec.value_dim * 4
        self.conv_bytes = (spec.conv_taps - 1) * self.channels * 4
        self.proj = self.out = None
        if not fused:
            self.proj, self.out = Linear(self.input_rows, rt), Linear(self.out_weight, rt)

    def state_bytes(self) -> int:
        return self.matrix_bytes + self.conv_bytes

    def inner(self, y: torch.Tensor, x: torch.Tensor, ctx, binding, scale: float = 1.0,
              out: torch.Tensor | None = None) -> torch.Tensor:
        """y: this mixer's columns of the projection of x, [q | k | v | a1 h | g1 h].  Returns [T, heads * value_dim] * scale."""
        s, ops = self.spec, self.rt.ops
        H, G, D, V, C = s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim, self.channels
        matrices = dataclasses.replace(binding, state=binding.state[:, :self.matrix_bytes])
        if s.conv_taps > 1:
            carried = dataclasses.replace(binding, state=binding.state[:, self.matrix_bytes:self.matrix_bytes + self.conv_bytes])
        else:
            carried = matrices                      # nothing is carried; the kernel wants a slot all the same
        conv = ops.short_conv_silu(y[:, :C], self.taps, ctx, carried)                        # float32 [T, C]
        z = self.decay_up(y[:, C:C + self.decay_rank].contiguous(), out_dtype=torch.float32)  # decay logits, float32 from here on
        gate = self.gate_up(y[:, C + self.decay_rank:C + self.decay_rank + self.gate_rank].contiguous())
        b = self.beta(x, out_dtype=torch.float32)
        prepared, beta = ops.delta_prepare(conv[:, :G * D], conv[:, G * D:2 * G * D], z, self.dt_bias, self.a_log, b,
                                           heads=H, kv_heads=G, dim=D, unit_eps=s.unit_eps, q_scale=s.q_scale)
        o = ops.recurrence_scan(prepared, conv[:, 2 * G * D:], ctx, matrices, heads=H, dim=D, vdim=V, beta=beta)
        return ops.head_norm_gate(o, gate, self.norm_weight, H, V, s.out_norm_eps, x.dtype, gate_kind="sigmoid",
                                  scale=scale, out=out)

    def forward(self, x: torch.Tensor, ctx, binding) -> torch.Tensor:
        return self.out(self.inner(self.proj(x), x, ctx, binding))
