"""
Mixers side by side on one input: y = sum_b scale_b * mixer_b(h).

Each branch is a mixer of its own kind that also exposes what lies between its projections
(`input_rows`: the stacked weights that read h; `inner(y, x, ctx, binding, scale, out)`: from its
columns of the fused projection to the input of its output projection, times `scale`; `out_weight`).
The branches' input projections run as one product and so do their output projections,

    [y_1 | y_2 | ...] = h . [W_1; W_2; ...]^T        y = [s_1 inner_1 | s_2 inner_2 | ...] . [O_1 | O_2 | ...]^T

so the weighted sum costs nothing of its own.  At most one branch keeps keys and values (it gets
the cache entry's pages); the branches' states are laid one behind the other in the entry's slot.
"""

from __future__ import annotations

import dataclasses
import inspect

import torch

from tinyserve_llm_b200.config.spec import ParallelMixerSpec
from tinyserve_llm_b200.parts.base import KVNeed, Mixer, Runtime, TensorDecl, part_class, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows

STATE_ALIGN = 256


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    @classmethod
    def declare(cls, spec: ParallelMixerSpec) -> dict[str, TensorDecl]:
        if not spec.branches:
            raise ValueError("a parallel mixer needs at least one branch")
        out: dict[str, TensorDecl] = {}
        for part, prefix, _ in spec.branches:
            for name, decl in part_class("mixer", part).declare(part).items():
                out[prefix + name] = decl
        return out

    def __init__(self, spec: ParallelMixerSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        self.branches, self.scales = [], []
        for part, prefix, scale in spec.branches:
            cls = part_class("mixer", part)
            sub = {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}
            if "fused" not in inspect.signature(cls.__init__).parameters:
                raise NotImplementedError(f"a {part.kind} mixer cannot be a branch of a parallel mixer: it does not expose "
                                          "its input rows, inner part and output weight")
            self.branches.append(cls(part, sub, rt, fused=True))
            self.scales.append(float(scale))
        if sum(b.kv_need() is not None for b in self.branches) > 1:
            raise NotImplementedError("at most one branch of a parallel mixer may keep keys and values")
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)
        self.proj = Linear(fuse_rows([b.input_rows for b in self.branches]), rt)
        self.out = Linear(torch.cat([b.out_weight for b in self.branches], dim=1).contiguous(), rt)
        self.in_offsets, self.inner_offsets, self.state_offsets = [0], [0], [0]
        for b in self.branches:
            self.in_offsets.append(self.in_offsets[-1] + b.input_rows.shape[0])
            self.inner_offsets.append(self.inner_offsets[-1] + b.inner_width)
            self.state_offsets.append(self.state_offsets[-1] + -(-int(b.state_bytes()) // STATE_ALIGN) * STATE_ALIGN)
        for b in self.branches:
            b.input_rows = b.out_weight = None          # the fused weights are the ones that stay

    def kv_need(self) -> KVNeed | None:
        return next((b.kv_need() for b in self.branches if b.kv_need() is not None), None)

    def state_bytes(self) -> int:
        return self.state_offsets[-1]

    def forward(self, x: torch.Tensor, ctx, binding) -> torch.Tensor:
        y = self.proj(x)
        inner = torch.empty((x.shape[0], self.inner_offsets[-1]), dtype=x.dtype, device=x.device)
        for i, (branch, scale) in enumerate(zip(self.branches, self.scales)):
            own = binding
            lo, size = self.state_offsets[i], int(branch.state_bytes())
            if binding is not None and binding.state is not None:
                own = dataclasses.replace(binding, state=binding.state[:, lo:lo + size] if size else None)
            branch.inner(y[:, self.in_offsets[i]:self.in_offsets[i + 1]], x, ctx, own, scale,
                         inner[:, self.inner_offsets[i]:self.inner_offsets[i + 1]])
        return self.out(inner)
