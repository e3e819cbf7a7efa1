"""
Plain, slow implementation of the Nipizen decoder in float64, one function per mechanism, written
from the design's equations.  It shares no code with the engine: tensors come in as a dict by their
checkpoint names, the configuration as the dict config.json holds.  Recurrences walk token by token.

    x_0 = embed[token]
    layer:  x <- x + mixer(LN1(x));  x <- x + moe(LN2(x))          LN: layer norm with weight, no bias
    mixer "parallel": left_scale * gated_attention(h) + right_scale * gated_delta_rule(h)
    mixer "mlstm":    matrix memory with exponential input gate and a running maximum
    logits = embed . LN_final(x)
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w


def rms_div(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotary_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """(frequencies [dims / 2], factor on cos and sin) of a rotation with optional YaRN rescaling."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turns_to_dim(t: float) -> float:
        return dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))

    lo = max(math.floor(turns_to_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turns_to_dim(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, dim]: channel i of the first rot dims is paired with i + dims / 2."""
    dims = int(rot["dims"])
    freq, mult = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = (ang.cos() * mult)[:, None, :], (ang.sin() * mult)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def gated_attention(h: torch.Tensor, w: dict, m: dict, eps: float, start: int = 0) -> torch.Tensor:
    """The left half of the parallel mixer over a whole sequence.  h [T, width]; w: tensors under '<layer>.mix.left.'."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = h @ w["q"].T + w["q.b"]
    k = h @ w["k"].T + w["k.b"]
    v = h @ w["v"].T + w["v.b"]
    q = rms_div(q, eps) * w["q.norm"]
    k = rms_div(k, eps) * w["k.norm"]
    pos = torch.arange(start, start + T)
    q = rotate(q.view(T, H, D), pos, m["rot"])
    k = rotate(k.view(T, G, D), pos, m["rot"])
    v = v.view(T, G, V)
    out = torch.zeros(T, H, V, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(m["scale"])
        mask = torch.ones(T, T, dtype=torch.bool).tril()
        s = s.masked_fill(~mask, -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    gated = out.reshape(T, H * V) * torch.sigmoid(h @ w["g"].T)
    return gated @ w["o"].T


def short_conv_silu(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]: y_t = sum_j taps[:, j] x_(t - (K - 1 - j)), zeros before the start; then silu."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j]
    return y * torch.sigmoid(y)


def gated_delta_rule(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """The right half of the parallel mixer.  w: tensors under '<layer>.mix.right.'."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = short_conv_silu(h @ w["q"].T, w["q.conv"]).view(T, G, D)
    k = short_conv_silu(h @ w["k"].T, w["k.conv"]).view(T, G, D)
    v = short_conv_silu(h @ w["v"].T, w["v.conv"]).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)                                     # [T, H]
    z = (h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]
    decay = torch.exp(-torch.exp(w["A_log"])[None, :, None] * torch.nn.functional.softplus(z).view(T, H, D))
    gate = torch.sigmoid((h @ w["g1"].T) @ w["g2"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(D, V, dtype=F64)
        for t in range(T):
            S = decay[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    out = rms_div(out, eps) * w["norm"] * gate
    return out.reshape(T, H * V) @ w["o"].T


def parallel_mixer(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    left = gated_attention(h, _under(w, "left."), m["left"], eps)
    right = gated_delta_rule(h, _under(w, "right."), m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def mlstm(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, V)
    i_gate = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    f_gate = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    out = torch.zeros(T, H, V, dtype=F64)
    for head in range(H):
        S = torch.zeros(D, V, dtype=F64)
        n = torch.zeros(D, dtype=F64)
        mx = torch.zeros((), dtype=F64)
        for t in range(T):
            new = torch.maximum(f_gate[t, head] + mx, i_gate[t, head])
            keep, take = torch.exp(f_gate[t, head] + mx - new), torch.exp(i_gate[t, head] - new)
            S = keep * S + take * torch.outer(k[t, head], v[t, head])
            n = keep * n + take * k[t, head]
            mx = new
            denom = torch.maximum((n @ q[t, head]).abs(), torch.exp(-mx)) + 1e-6
            out[t, head] = (S.T @ q[t, head]) / denom
    out = rms_div(out, eps).reshape(T, H * V) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def routed_experts(h: torch.Tensor, w: dict, f: dict) -> torch.Tensor:
    """Sigmoid scores, the `top` largest chosen, the score multiplies the expert's input; expert: down(relu(up x)^2)."""
    experts, top = int(f["router"]["experts"]), int(f["router"]["top"])
    scores = torch.sigmoid(h @ w["router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(scores[t, e]), e))[:top]
        for e in order:
            x = scores[t, e] * h[t]
            out[t] = out[t] + w[f"e{e}.down"] @ torch.relu(w[f"e{e}.up"] @ x) ** 2
    return out


def _under(w: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], return_layers: bool = False):
    """float64 logits [T, vocab] of one sequence from its start (and the stream after every layer, if asked)."""
    w = {k: v.to(F64) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    after = []
    for i, layer in enumerate(config["layers"]):
        lw = _under(w, f"l{i}.")
        h = layer_norm(x, lw["norm1"], eps)
        mixers = {"parallel": parallel_mixer, "mlstm": mlstm}
        x = x + mixers[layer["type"]](h, _under(lw, "mix."), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            h = layer_norm(x, lw["norm2"], eps)
            x = x + routed_experts(h, _under(lw, "mlp."), layer["mlp"])
        after.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
