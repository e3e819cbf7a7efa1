"""
Plain, slow implementation of the Duduvik decoder, one function per mechanism, in float64 on the
CPU, token by token where the design is a recurrence.  It is the oracle of the tests and shares no
code with the engine: it takes the raw config.json dictionary and a dictionary of tensors by their
checkpoint names.

Notation: h is a sublayer's input [T, width]; p_t the position of token t in its sequence.
"""

from __future__ import annotations

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """
    x [T, heads, d]: the first `dims` channels of each head are turned, channel i with channel
    i + dims/2, by the angle p * base^(-2i/dims); the other channels pass.
    """
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    angle = positions.double()[:, None] * freq[None, :]                 # [T, half]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., dims:]), dim=-1)


# ---------------------------------------------------------------------------------------------- mixers
def mixer_gla(m: dict, w: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Gated linear attention with a decay per key channel; state S [heads, dim, vdim] from zero."""
    H, D, V, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, V)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    out = []
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    o = torch.stack(out)                                               # [T, H, V]
    o = norm_plain(o, w["norm"], eps).reshape(T, H * V)
    g = h @ w["g"].T
    return (o * (g * torch.sigmoid(g))) @ w["o"].T


def mixer_retention(m: dict, w: dict, h: torch.Tensor, positions: torch.Tensor, eps: float) -> torch.Tensor:
    """Linear attention with one fixed decay per head, rotary q and k, no softmax, no denominator."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rotate_half((h @ w["q"].T).view(T, H, D), positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half((h @ w["k"].T).view(T, H, D), positions, m["rot"]["dims"], m["rot"]["base"]) * D ** -0.5
    v = (h @ w["v"].T).view(T, H, V)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    out = []
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    o = rms_unit(torch.stack(out), eps).reshape(T, H * V)
    g = h @ w["g"].T
    return (o * (g * torch.sigmoid(g))) @ w["o"].T


def mixer_latent_attention(m: dict, w: dict, h: torch.Tensor, positions: torch.Tensor, eps: float) -> torch.Tensor:
    """Softmax attention whose keys and values come from a shared latent, with one rotated key part for all heads."""
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    cq = norm_plain(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, D + R)
    q_flat, q_rot = q[..., :D], rotate_half(q[..., D:], positions, m["rot"]["dims"], m["rot"]["base"])
    kv = h @ w["dkv"].T
    c = norm_plain(kv[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate_half(kv[:, None, rank:], positions, m["rot"]["dims"], m["rot"]["base"])[:, 0]     # [T, R]
    k_flat = (c @ w["uk"].T).view(T, H, D)
    val = (c @ w["uv"].T).view(T, H, V)
    window = m["mask"]["size"]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        lo = max(0, t - window + 1)
        s = (torch.einsum("hd,jhd->hj", q_flat[t], k_flat[lo:t + 1])
             + torch.einsum("hr,jr->hj", q_rot[t], k_rot[lo:t + 1])) * m["scale"]
        p = torch.softmax(s, dim=-1)
        out[t] = torch.einsum("hj,jhv->hv", p, val[lo:t + 1])
    return out.reshape(T, H * V) @ w["o"].T


# ---------------------------------------------------------------------------------------------- feed-forward
def ff_dense(w: dict, h: torch.Tensor) -> torch.Tensor:
    return (torch.relu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def ff_expert(w: dict, prefix: str, h: torch.Tensor, limit: float) -> torch.Tensor:
    g = (h @ w[prefix + "gate"].T).clamp(max=limit)
    u = (h @ w[prefix + "up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].T


def ff_moe(f: dict, w: dict, h: torch.Tensor) -> torch.Tensor:
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ w["router"].T + w["router.b"]
    best, which = z.topk(top, dim=-1)
    share = torch.softmax(best, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(which[t, j])
            out[t] += share[t, j] * ff_expert(w, f"e{e}.", h[t:t + 1], f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + ff_expert(w, "shared.", h, f["shared"]["limit"])
    return out


# ---------------------------------------------------------------------------------------------- the model
def _sub(w: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, ids: list[int], return_layers: bool = False):
    """Logits [T, vocab] of one sequence from position 0 (and the stream after every layer, if asked)."""
    w = {k: v.double() for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    positions = torch.arange(len(ids))
    x = w["embed"][torch.tensor(ids)] * config["embedding"]["scale"]
    layers = []
    for i, layer in enumerate(config["layers"]):
        lw = _sub(w, f"l{i}.")
        h = norm_around_zero(x, lw["norm1"], eps)
        mw = _sub(lw, "mix.")
        if layer["type"] == "gla":
            y = mixer_gla(layer["mixer"], mw, h, eps)
        elif layer["type"] == "retention":
            y = mixer_retention(layer["mixer"], mw, h, positions, eps)
        elif layer["type"] == "latent_attention":
            y = mixer_latent_attention(layer["mixer"], mw, h, positions, eps)
        else:
            raise ValueError(layer["type"])
        x = x + norm_around_zero(y, lw["norm1b"], eps)
        f = layer.get("mlp")
        if f is not None:
            h = norm_around_zero(x, lw["norm2"], eps)
            fw = _sub(lw, "mlp.")
            y = ff_dense(fw, h) if f["kind"] == "dense" else ff_moe(f, fw, h)
            x = x + norm_around_zero(y, lw["norm2b"], eps)
        layers.append(x)
    logits = norm_around_zero(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(layers)) if return_layers else logits
