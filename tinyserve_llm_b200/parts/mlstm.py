"""
Matrix memory with exponential gating (the mLSTM of xLSTM): per head a matrix S and a vector n of
decayed keys, stabilised by a running maximum m of the log gates.

    q = W_q h * q_scale, k = W_k h, v = W_v h
    i = cap tanh((W_i h + b_i) / cap)            f = log_sigmoid(cap tanh((W_f h + b_f) / cap))
    m_t = max(f + m_(t-1), i)                    (m starts at 0)
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T,   n_t likewise with k alone
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + denominator_eps)
    y = W_o ( concat(o / rms(o)) * w * sigmoid(W_g h) )

This is the linear recurrence of `linear_recurrence.cu` with one decay per head and token, keys
scaled by exp(i - m_t), and one more value column that is constantly 1: that column of the state is
n, and the same column of the read-out is n . q.  A small kernel walks the gates and the maximum in
order; the scan and the state slot are the framework's.  The state (float32) holds
[heads, key_dim, value_dim + 1] and then the heads' maxima.  The gates' projection leaves its
product in float32.
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import MatrixLSTMSpec
from tinyserve_llm_b200.parts.base import Mixer, Runtime, TensorDecl, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows

MAX_KEY_DIM = 256       # csrc/linear_recurrence.cu


@register_part("mixer", "mlstm")
class MatrixLSTM(Mixer):
    graph_safe = True

    @classmethod
    def validate(cls, spec: MatrixLSTMSpec) -> None:
        if not 0 < spec.key_dim <= MAX_KEY_DIM:
            raise ValueError(f"key_dim={spec.key_dim} is not supported: the recurrence kernel takes up to {MAX_KEY_DIM}")
        if spec.gate_cap <= 0:
            raise ValueError(f"gate_cap={spec.gate_cap} must be positive")

    @classmethod
    def declare(cls, spec: MatrixLSTMSpec) -> dict[str, TensorDecl]:
        cls.validate(spec)
        qk, vv, hidden, H = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim, spec.hidden_size, spec.num_heads
        return {
            "q": TensorDecl((qk, hidden)), "k": TensorDecl((qk, hidden)), "v": TensorDecl((vv, hidden)),
            "g": TensorDecl((vv, hidden)), "o": TensorDecl((hidden, vv)), "norm": TensorDecl((vv,), init="unit"),
            "i": TensorDecl((H, hidden)), "i.b": TensorDecl((H,)), "f": TensorDecl((H, hidden)), "f.b": TensorDecl((H,)),
        }

    def __init__(self, spec: MatrixLSTMSpec, tensors: dict[str, torch.Tensor], rt: Runtime, fused: bool = False) -> None:
        super().__init__(spec, tensors, rt)
        self.validate(spec)
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.input_rows = fuse_rows([tensors["q"], tensors["k"], tensors["v"], tensors["g"]])
        self.out_weight = tensors["o"]
        self.inner_width = spec.num_heads * spec.value_dim
        self.gates = Linear(fuse_rows([tensors["i"], tensors["f"]]), rt)
        self.bias_i = tensors["i.b"].to(**f32).contiguous()
        self.bias_f = tensors["f.b"].to(**f32).contiguous()
        self.norm_weight = tensors["norm"].to(**f32).contiguous()
        self.matrix_floats = spec.num_heads * spec.key_dim * (spec.value_dim + 1)
        self.proj = self.out = None
        if not fused:
            self.proj, self.out = Linear(self.input_rows, rt), Linear(self.out_weight, rt)

    def state_bytes(self) -> int:
        return (self.matrix_floats + self.spec.num_heads) * 4

    def inner(self, y: torch.Tensor, x: torch.Tensor, ctx, binding, scale: float = 1.0,
              out: torch.Tensor | None = None) -> torch.Tensor:
        """y: this mixer's columns of the projection of x, [q | k | v | g].  Returns [T, heads * value_dim] * scale."""
        s, ops = self.spec, self.rt.ops
        H, D, V = s.num_heads, s.key_dim, s.value_dim
        q, k, v, g = y[:, :H * D], y[:, H * D:2 * H * D], y[:, 2 * H * D:2 * H * D + H * V], y[:, 2 * H * D + H * V:2 * H * D + 2 * H * V]
        gates = self.gates(x, out_dtype=torch.float32)                    # [T, 2 H]: input gates, forget gates
        prepared, log_max = ops.mlstm_prepare(q, k, gates, self.bias_i, self.bias_f, ctx, binding, heads=H, dim=D,
                                              cap=s.gate_cap, q_scale=s.q_scale, max_offset_floats=self.matrix_floats)
        o = ops.recurrence_scan(prepared, v, ctx, binding, heads=H, dim=D, vdim=V + 1, v_cols=V)    # column V: n . q
        return ops.head_norm_gate(o, g, self.norm_weight, H, V, s.out_norm_eps, x.dtype, gate_kind="sigmoid",
                                  weight_per_head=True, log_max=log_max, scale=scale, out=out)

    def forward(self, x: torch.Tensor, ctx, binding) -> torch.Tensor:
        return self.out(self.inner(self.proj(x), x, ctx, binding))
