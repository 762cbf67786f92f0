"""A plain, slow implementation of the Niduvik design: one function per mechanism, written from the
design's equations with torch on the CPU (float64 unless told otherwise).  It is the oracle of the
tests and shares no code with the engine: it reads the configuration as a plain dict and the weights
as a dict of tensors under their checkpoint names, runs one whole sequence at a time, token by token
where the design is a recurrence, and keeps nothing between calls.

Notation: T tokens, W width, H query heads, G key/value heads (or groups), d the query/key size of a
head, e the value size, N the state size of the recurrence."""
from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) (* weight) over the last dimension."""
    y = x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance-bias table for a key n tokens back: one row a distance below rows // 2, then rows
    spaced evenly in the logarithm of the distance up to `far`, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    """Whether the query at position i sees the key at position j."""
    return j <= i and (i - j < size or j < keep_first)


def attention_scores(q, k, rel, scale, softcap, far, size, keep_first):
    """q [T, H, d], k [T, G, d], rel [rows, H] -> scores [H, T, T] with -inf where a key is not seen."""
    T, H, _ = q.shape
    G = k.shape[1]
    rows = rel.shape[0]
    back = torch.arange(T)[:, None] - torch.arange(T)[None, :]                       # i - j
    seen = torch.tensor([[visible(i, j, size, keep_first) for j in range(T)] for i in range(T)])
    row_of = torch.tensor([distance_bucket(n, rows, far) for n in range(T)])[back.clamp(min=0)]
    s = torch.full((H, T, T), -math.inf, dtype=q.dtype)
    for h in range(H):
        raw = (q[:, h] @ k[:, h // (H // G)].T) * scale
        raw = softcap * torch.tanh(raw / softcap) + rel[row_of, h]
        s[h] = torch.where(seen, raw, s[h])
    return s


def sink_softmax(s: torch.Tensor) -> torch.Tensor:
    """exp(s_j) / (1 + sum_j exp(s_j)) over the last dimension: a sink with score 0 and no value."""
    m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(dim=-1, keepdim=True))


def attention_mixer(h, w, prefix, c, v_first):
    """h [T, W] -> (output [T, W], this layer's values before mixing [T, G, e]).  `v_first`: the values of
    the first layer that mixes values (None in that layer and in layers that do not mix)."""
    H, G, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = (h @ w[prefix + "q"].T + w[prefix + "q.b"]).view(T, H, d)
    k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).view(T, G, d)
    v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).view(T, G, e)
    own = v
    if c.get("v_mix") and v_first is not None:
        lam = w[prefix + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    s = attention_scores(q, k, w[prefix + "rel"], c["scale"], c["softcap"], c["bias_max"], c["mask"]["size"],
                         c["mask"]["keep_first"])
    p = sink_softmax(s)
    gate = torch.sigmoid(h @ w[prefix + "g"].T)                      # [T, H]
    out = torch.empty(T, H, e, dtype=h.dtype)
    for head in range(H):
        out[:, head] = (p[head] @ v[:, head // (H // G)]) * gate[:, head:head + 1]
    return out.reshape(T, H * e) @ w[prefix + "o"].T, own


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], weight [C, taps] (last column: the current token), zeros before the start."""
    T, C = x.shape
    taps = weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    out = bias.expand(T, C).clone()
    for k in range(taps):
        out = out + padded[k:k + T] * weight[:, k]
    return out


def selective_scan(x, B, C, dt_raw, dt_bias, A_log, D):
    """x [T, heads, e], B and C [T, G, N], dt_raw [T, heads] -> y [T, heads, e]; the state starts at zero."""
    T, heads, e = x.shape
    G, N = B.shape[1], B.shape[2]
    dt = torch.nn.functional.softplus(dt_raw + dt_bias, threshold=1e9)
    decay = torch.exp(-torch.exp(A_log) * dt)
    S = torch.zeros(heads, N, e, dtype=x.dtype)
    y = torch.empty(T, heads, e, dtype=x.dtype)
    for t in range(T):
        for head in range(heads):
            g = head // (heads // G)
            S[head] = decay[t, head] * S[head] + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S[head].T @ C[t, g] + D[head] * x[t, head]
    return y


def gated_part_norm(y, z, weight, parts, eps):
    """(y * silu(z)), each of `parts` equal parts of a row by its own root mean square, times weight."""
    T, inner = y.shape
    g = y * silu(z)
    return rms_norm(g.view(T, parts, inner // parts), None, eps).reshape(T, inner) * weight


def mamba2_mixer(h, w, prefix, c, eps):
    """h [T, W] -> [T, W]: the recurrence token by token, state from zero."""
    heads, e, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = heads * e
    T = h.shape[0]
    proj = h @ w[prefix + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].view(T, heads, e)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    y = selective_scan(x, B, C, dt, w[prefix + "dt_bias"], w[prefix + "A_log"], w[prefix + "D"])
    y = gated_part_norm(y.reshape(T, inner), z, w[prefix + "norm"], c["norm_groups"], eps)
    return y @ w[prefix + "o"].T


def clamped_glu(g, u, limit, slope=1.702):
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, min=-limit, max=limit)
    return g * torch.sigmoid(slope * g) * (u + 1.0)


def feed_forward(h, w, prefix, c):
    return clamped_glu(h @ w[prefix + "gate"].T, h @ w[prefix + "up"].T, c["limit"]) @ w[prefix + "down"].T


def forward(config: dict, weights: dict, tokens, dtype=torch.float64):
    """One whole sequence: (logits [T, vocab], the stream after every layer [layers, T, W])."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    v_first = None
    streams = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            a, own = attention_mixer(h, w, p + "mix.", layer["mixer"], v_first)
            if layer["mixer"].get("v_mix") and v_first is None:
                v_first = own
        elif layer["type"] == "mamba2":
            a = mamba2_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(a, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            f = feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
            x = x + rms_norm(f, w[p + "norm2b"], eps)
        streams.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    return logits, torch.stack(streams)
