"""A plain, slow restatement of the Vezalorn design in torch on the CPU: one
function per mechanism, whole sequences at once, no cache, no batching. It
shares no code with the package and is what the package's kernels, cache and
step function are compared with.

Notation: h is a [T, width] matrix of one sequence's tokens (positions 0..T-1),
W a matrix stored [out, in] and applied as h @ W.T. All arithmetic runs in the
element type of the tensors given (float64 in the tests).
"""
from __future__ import annotations

import math

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(v, eps):
    """v divided by its root mean square over the last axis, eps under the root."""
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def group_rms_norm(v, w, groups: int, eps: float):
    """The last axis in `groups` equal consecutive parts, each divided by its own root mean square; then times w."""
    T, n = v.shape
    parts = v.reshape(T, groups, n // groups)
    return unit_rms(parts, eps).reshape(T, n) * w


def rotate_pairs(v, positions, base: float, dims: int):
    """v [T, ..., d]: of the last axis' first `dims` values, (2i, 2i+1) turn by positions * base^(-2i/dims)."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=v.dtype)
    freq = torch.as_tensor(base, dtype=v.dtype) ** (-2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_attention(h, w, p, eps):
    """w: q, dkv, dkv.norm, uk, uv, o. p: heads, dim, rot_dim, vdim, kv_rank, scale, rot{base, dims}."""
    T = h.shape[0]
    H, d, r, vd, rank = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w["q"].T).reshape(T, H, d + r)
    q_plain, q_turn = q[..., :d], rotate_pairs(q[..., d:], pos, p["rot"]["base"], p["rot"]["dims"])
    down = h @ w["dkv"].T
    c = unit_rms(down[:, :rank], eps) * w["dkv.norm"]
    k_turn = rotate_pairs(down[:, rank:], pos, p["rot"]["base"], p["rot"]["dims"])      # [T, r], one for all heads
    k_plain = (c @ w["uk"].T).reshape(T, H, d)
    v = (c @ w["uv"].T).reshape(T, H, vd)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_turn, k_turn)) * p["scale"]
    hidden = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    scores = scores.masked_fill(hidden, float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    o = torch.einsum("hij,jhv->ihv", weights, v).reshape(T, H * vd)
    return o @ w["o"].T


def mingru(h, w, state=None):
    """w: z, z.b, x, x.b, g, o. Returns (output [T, width], the state after the last token)."""
    z = torch.sigmoid(h @ w["z"].T + w["z.b"])
    u = h @ w["x"].T + w["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = h @ w["g"].T
    gate = gate * torch.sigmoid(gate)
    S = torch.zeros(z.shape[1], dtype=h.dtype) if state is None else state
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S)
    return (torch.stack(rows) * gate) @ w["o"].T, S


def dense_mlp(h, w):
    """w: gate, gate.b, up, up.b, down, down.b."""
    return (gelu_tanh(h @ w["gate"].T + w["gate.b"]) * (h @ w["up"].T + w["up.b"])) @ w["down"].T + w["down.b"]


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence. `layers_out`, a list, receives the stream after every layer."""
    t = {k: v.to(dtype) for k, v in tensors.items()}
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        if layer["type"] == "latent_attention":
            m = latent_attention(x, sub(t, pre + "mix."), layer["mixer"], eps)
        elif layer["type"] == "mingru":
            m, _ = mingru(x, sub(t, pre + "mix."))
        else:
            raise ValueError(layer["type"])
        m = m * torch.sigmoid(x @ t[pre + "rg1"].T + t[pre + "rg1.b"])
        x = x + group_rms_norm(m, t[pre + "norm1"], groups, eps)
        if layer.get("mlp") is not None:
            f = dense_mlp(x, sub(t, pre + "mlp."))
            f = f * torch.sigmoid(x @ t[pre + "rg2"].T + t[pre + "rg2.b"])
            x = x + group_rms_norm(f, t[pre + "norm2"], groups, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return group_rms_norm(x, t["final.norm"], groups, eps) @ t["embed"].T
