"""A plain restatement of the Tufadra design in 64-bit torch: whole sequences, no cache, no batching, one function per
mechanism. It shares no code with the package and is slow on purpose.

Notation: T tokens, width H. A layer: h = N(x); x <- x + A(h) + F(h), where N divides by the root mean square and
multiplies by 1 + w, A is causal attention without a rotation (queries and keys normed over the whole projection, a
query temperature that grows with the position, values of a width of their own) and F a mixture of experts beside one
shared expert. The embedding adds a learned vector per position; the logits are products with the embedding table."""
import math

import torch


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """x / rms(x) * (1 + w): the stored weight lies around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_exact(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def embed_with_positions(table, pos_table, tokens):
    T = len(tokens)
    return table[torch.as_tensor(tokens, dtype=torch.long)] + pos_table[:T]


def query_temperature(T, coef, every):
    """The factor of the query at positions 0..T-1: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(T, dtype=torch.float64)
    return 1.0 + coef * torch.log(torch.floor((p + 1.0) / every) + 1.0)


def causal_attention(q, k, v, scale, weights_out=None):
    """q [T, nh, d], k [T, nkv, d], v [T, nkv, dv]: query head h reads key/value head h // (nh / nkv); position i sees
    every j <= i; ordinary softmax. Returns [T, nh, dv]."""
    T, nh, _ = q.shape
    per = nh // k.shape[1]
    hidden = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
    out = torch.zeros(T, nh, v.shape[-1], dtype=torch.float64)
    for h in range(nh):
        s = (q[:, h] @ k[:, h // per].T) * scale
        p = torch.softmax(s.masked_fill(hidden, float("-inf")), -1)
        if weights_out is not None:
            weights_out.append(p)
        out[:, h] = p @ v[:, h // per]
    return out


def attention(h, w, prefix, m, eps, weights_out=None):
    T = h.shape[0]
    q, k, v = h @ w[prefix + "q"].T, h @ w[prefix + "k"].T, h @ w[prefix + "v"].T
    q = unit_rms(q, eps) * w[prefix + "q.norm"]          # over all heads at once, plain weights
    k = unit_rms(k, eps) * w[prefix + "k.norm"]
    if m.get("q_temp") is not None:
        q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None]
    o = causal_attention(q.reshape(T, m["heads"], m["dim"]), k.reshape(T, m["kv_heads"], m["dim"]),
                         v.reshape(T, m["kv_heads"], m["vdim"]), m["scale"], weights_out)
    return o.reshape(T, -1) @ w[prefix + "o"].T


def route(z, correction, top, groups, scale):
    """z [T, E] router sums. Returns (chosen experts [T, top] by descending choice score, their weights [T, top])."""
    T, E = z.shape
    s = torch.sigmoid(z)
    c = s + correction
    if groups is not None and groups["count"] > 1:
        n, size = groups["count"], E // groups["count"]
        by_group = c.reshape(T, n, size)
        score = by_group.sort(-1, descending=True).values[..., :2].sum(-1)      # a group of one has one score
        kept = torch.zeros(T, n, dtype=torch.bool)
        for t in range(T):
            order = sorted(range(n), key=lambda g: (-float(score[t, g]), g))
            kept[t, order[:groups["keep"]]] = True
        c = by_group.masked_fill(~kept[:, :, None], float("-inf")).reshape(T, E)
    chosen = torch.zeros(T, top, dtype=torch.long)
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(c[t, e]), e))
        chosen[t] = torch.tensor(order[:top])
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20) * scale


def expert(h, up, down):
    return gelu_exact(h @ up.T) @ down.T


def mixture(h, w, prefix, f):
    r = f["router"]
    chosen, weights = route(h @ w[prefix + "router"].T, w[prefix + "correction"], r["top"], r.get("groups"), r["scale"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            out[t] += a * expert(h[t], w[f"{prefix}e{e}.up"], w[f"{prefix}e{e}.down"])
    if f.get("shared") is not None:
        gate = torch.sigmoid(h @ w[prefix + "shared.sg"].T)
        out = out + gate * expert(h, w[prefix + "shared.up"], w[prefix + "shared.down"])
    return out


def forward(cfg, tensors, tokens, layers_out=None):
    """Logits [T, vocab] (float64) for one sequence. `layers_out`: a list that gets the stream after every layer."""
    w = {k: v.double() for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = embed_with_positions(w["embed"], w["pos"], tokens)
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of")
        while src is not None and cfg["layers"][src].get("weights_of") is not None:
            src = cfg["layers"][src]["weights_of"]
        p = f"l{i if src is None else src}."
        h = offset_norm(x, w[p + "norm1"], eps)
        y = attention(h, w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + mixture(h, w, p + "mlp.", layer["mlp"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["embed"].T
