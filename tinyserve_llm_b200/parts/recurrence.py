"""
Linear attention as a recurrence over a per-request matrix state (retention, gated linear attention).

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t          per head, S [key_dim, value_dim]
    y   = W_o ( norm_heads(o) * silu(W_g h) )

The state lives in the request's fixed-size slot of the cache manager (float32, zeroed at admission,
given back at release), so prompts in portions, decoding and mixed batches are one code path: the
kernel reads the slot, walks over the request's tokens of the step and writes the slot back.

The decay a_t is, by `spec.decay`:
  "head"            one constant per head (`spec.head_decays`)
  "channel_logits"  per key channel, a = sigmoid(z)^(1/tau), z = W_a2 (W_a1 h) + b; the kernel takes
                    z in float32 and computes the power as exp(log_sigmoid(z) / tau)
q and k may be rotated (`spec.position`, rotate-half with angles computed in the kernel) and scaled
(`q_scale`, `k_scale`); both happen in float32 on the way into the recurrence.

Tensors (local names): q, k, v, g, o, and for "channel_logits" a1, a2, a2.b; `norm` (one weight per
value channel, shared by the heads) if the output norm has one.
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import LinearRecurrenceSpec
from tinyserve_llm_b200.parts.base import Mixer, Runtime, TensorDecl, part_class, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows

MAX_KEY_DIM = 256       # csrc/linear_recurrence.cu: 16 row groups x 16 rows in registers


@register_part("mixer", "linear_recurrence")
class LinearRecurrence(Mixer):
    graph_safe = True

    @classmethod
    def validate(cls, spec: LinearRecurrenceSpec) -> None:
        if spec.decay not in ("head", "channel_logits"):
            raise NotImplementedError(f"decay {spec.decay!r} is not supported; have ['head', 'channel_logits']")
        if spec.key_dim > MAX_KEY_DIM:
            raise ValueError(f"key_dim={spec.key_dim} is not supported: the recurrence kernel takes up to {MAX_KEY_DIM}")
        if spec.decay == "head" and len(spec.head_decays) != spec.num_heads:
            raise ValueError(f"{len(spec.head_decays)} decays for {spec.num_heads} heads")

    @classmethod
    def declare(cls, spec: LinearRecurrenceSpec) -> dict[str, TensorDecl]:
        cls.validate(spec)
        qk, vv, hidden = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim, spec.hidden_size
        out = {
            "q": TensorDecl((qk, hidden)), "k": TensorDecl((qk, hidden)), "v": TensorDecl((vv, hidden)),
            "g": TensorDecl((vv, hidden)), "o": TensorDecl((hidden, vv)),
        }
        if spec.decay == "channel_logits":
            rank = spec.decay_rank if spec.decay_rank > 0 else -1       # -1: the checkpoint's own size
            out.update({"a1": TensorDecl((rank, hidden)), "a2": TensorDecl((qk, rank)), "a2.b": TensorDecl((qk,))})
        if spec.out_norm_weight:
            out["norm"] = TensorDecl((spec.value_dim,), init="unit")
        return out

    def __init__(self, spec: LinearRecurrenceSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        self.validate(spec)
        # one projection for everything that reads h: columns [q | k | v | g | a1 h]
        rows = [tensors["q"], tensors["k"], tensors["v"], tensors["g"]]
        self.decay_rank = 0
        if spec.decay == "channel_logits":
            if tensors["a1"].shape[0] != tensors["a2"].shape[1]:
                raise ValueError(f"the decay projection's inner sizes differ: {tuple(tensors['a1'].shape)} and "
                                 f"{tuple(tensors['a2'].shape)}")
            self.decay_rank = int(tensors["a1"].shape[0])
            rows.append(tensors["a1"])
            self.decay_up = Linear(tensors["a2"], rt)
            self.decay_bias = tensors["a2.b"].to(device=rt.device, dtype=torch.float32).contiguous()
            self.head_decays = None
        else:
            self.head_decays = torch.tensor(spec.head_decays, dtype=torch.float32, device=rt.device)
        self.proj = Linear(fuse_rows(rows), rt)
        self.out = Linear(tensors["o"], rt)
        self.norm_weight = None
        if spec.out_norm_weight:
            self.norm_weight = tensors["norm"].to(device=rt.device, dtype=torch.float32).contiguous()
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position)(spec.position, {}, rt)
            if getattr(self.position, "frequencies", None) is None:
                raise NotImplementedError("the recurrence rotates q and k itself: it takes a position part with `frequencies`")

    def state_bytes(self) -> int:
        return self.spec.num_heads * self.spec.key_dim * self.spec.value_dim * 4

    def forward(self, x: torch.Tensor, ctx, binding) -> torch.Tensor:
        spec, ops = self.spec, self.rt.ops
        H, D, V = spec.num_heads, spec.key_dim, spec.value_dim
        y = self.proj(x)                                                  # [T, 2 H D + 2 H V (+ rank)]
        q, k, v, g = y[:, :H * D], y[:, H * D:2 * H * D], y[:, 2 * H * D:2 * H * D + H * V], y[:, 2 * H * D + H * V:2 * H * D + 2 * H * V]
        z = None
        if self.decay_rank:
            low = y[:, 2 * H * D + 2 * H * V:].contiguous()
            z = self.decay_up(low, out_dtype=torch.float32)               # decay logits, float32 from here on
        o = ops.linear_recurrence(q, k, v, ctx, binding, heads=H, dim=D, vdim=V, z=z,
                                  bias=self.decay_bias if self.decay_rank else None, head_decays=self.head_decays,
                                  inv_tau=1.0 / spec.tau, q_scale=spec.q_scale, k_scale=spec.k_scale,
                                  position=self.position)                 # float32 [T, H V]
        gated = ops.head_norm_gate(o, g, self.norm_weight, H, V, spec.out_norm_eps, x.dtype)
        return self.out(gated)
