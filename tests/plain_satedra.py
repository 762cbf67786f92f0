"""A plain, slow implementation of the Satedra design: one function per mechanism, written from the design's
equations with torch on the CPU (float64 unless told otherwise).  It is the oracle of the tests and shares no
code with the engine: it reads the configuration as a plain dict and the weights as a dict of tensors under
their checkpoint names, runs one whole sequence at a time and keeps nothing between calls.

Notation: T tokens, W width, H heads, d the unrotated and r the rotated query/key size of a head, e the value
size of a head, R the size of the latent, E routed experts, I identity experts."""
from __future__ import annotations

import math

import torch


def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * weight + bias over the last dimension; var is the mean squared deviation."""
    mean = x.mean(dim=-1, keepdim=True)
    var = (x - mean).pow(2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def rms_norm(x, weight, eps):
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def yarn_frequencies(dims: int, base: float, scaling: dict | None):
    """(frequencies [dims / 2], magnitude).  Without scaling f_i = base^(-2i/dims) and the magnitude is 1.  With
    it the frequencies of slow pairs are divided by the factor, those of fast pairs stay, a linear ramp between
    them; cosines and sines grow by 0.1 ln(factor) + 1."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return torch.tensor(f, dtype=torch.float64), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):            # the pair that makes `turns` turns over the original length
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, frequencies, magnitude, angle_dtype=torch.float64):
    """x [T, ..., dims]: element i pairs with element i + dims / 2; the pair (u, v) at position p becomes
    (u cos a - v sin a, v cos a + u sin a), a = p f_i, cos and sin times `magnitude`.  `angle_dtype`: the precision
    in which the table and the product p f_i are held (the design computes angles in 32-bit)."""
    half = frequencies.shape[0]
    angle = (positions.to(angle_dtype)[:, None] * frequencies.to(angle_dtype)[None, :]).to(torch.float64)          # [T, half]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (half,)
    cos = (torch.cos(angle) * magnitude).to(x.dtype).view(shape)
    sin = (torch.sin(angle) * magnitude).to(x.dtype).view(shape)
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., 2 * half:]], dim=-1)


def window_mask(T: int, size: int | None):
    """[T, T] bool: query i sees key j when 0 <= i - j < size (no size: every earlier key and itself)."""
    back = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    seen = back >= 0
    return seen & (back < size) if size else seen


def latent_keys(h, w, prefix, c, eps, positions):
    """What a latent-attention layer keeps of its input h [T, W]: the normed latent [T, R] and the rotated key
    part [T, r] that all heads share."""
    R, r = c["kv_rank"], c["rot_dim"]
    down = h @ w[prefix + "dkv"].T
    latent = rms_norm(down[:, :R], w[prefix + "dkv.norm"], eps)
    f, magnitude = yarn_frequencies(c["rot"]["dims"], c["rot"]["base"], c["rot"].get("scaling"))
    return latent, rotate(down[:, R:R + r], positions, f, magnitude)


def latent_attention(h, w, prefix, c, eps, kept, positions=None):
    """h [T, W] -> [T, W].  `kept` = (latent, rotated key part) of the layer whose cache this one reads (its own
    from `latent_keys`, or another layer's)."""
    T = h.shape[0]
    H, d, r, e = c["heads"], c["dim"], c["rot_dim"], c["vdim"]
    positions = torch.arange(T) if positions is None else positions
    latent, key_rot = kept
    q = (h @ w[prefix + "q"].T).view(T, H, d + r)
    f, magnitude = yarn_frequencies(c["rot"]["dims"], c["rot"]["base"], c["rot"].get("scaling"))
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], positions, f, magnitude)
    k_plain = (latent @ w[prefix + "uk"].T).view(T, H, d)
    v = (latent @ w[prefix + "uv"].T).view(T, H, e)
    seen = window_mask(T, (c.get("mask") or {}).get("size"))
    gate = torch.sigmoid(h @ w[prefix + "g"].T)                                   # [T, H]
    out = torch.empty(T, H, e, dtype=h.dtype)
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ key_rot.T) * c["scale"]
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        out[:, head] = (torch.softmax(s, dim=-1) @ v[:, head]) * gate[:, head:head + 1]
    return out.reshape(T, H * e) @ w[prefix + "o"].T


def gated_unit(h, w, prefix):
    """down(silu(gate h) * (up h))."""
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h, w, prefix, router):
    """(chosen [T, top] expert numbers, weights [T, top]).  Scores are a softmax over routed and identity
    experts; the choice adds a correction to the scores, the weights do not; weights are the chosen scores over
    their sum, times the router's scale."""
    scores = torch.softmax(h @ w[prefix + "router"].T, dim=-1)
    chosen = torch.topk(scores + w[prefix + "correction"], router["top"], dim=-1).indices
    picked = torch.gather(scores, 1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * router["scale"]


def mixture(h, w, prefix, c):
    """Routed experts (the last `identity` numbers hand their input on), plus a shared expert behind a sigmoid
    gate of one number a token."""
    router = c["router"]
    E = router["experts"]
    chosen, weights = route(h, w, prefix, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t].tolist(), weights[t]):
            y = gated_unit(h[t:t + 1], w, f"{prefix}e{e}.")[0] if e < E else h[t]
            out[t] += weight * y
    if c.get("shared"):
        out = out + torch.sigmoid(h @ w[prefix + "shared.sg"].T) * gated_unit(h, w, prefix + "shared.")
    return out


def forward(config: dict, w: dict, tokens, dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] of one sequence from position 0.  `layers_out`: a list that gets the residual stream
    after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        c = layer["mixer"]
        if layer["type"] != "latent_attention":
            raise ValueError(f"layer type {layer['type']!r}")
        source = c.get("kv_from")
        kept[i] = latent_keys(h, w, p + "mix.", c, eps, positions) if source is None else kept[source]
        x = x + latent_attention(h, w, p + "mix.", c, eps, kept[i], positions)
        if layer.get("mlp") is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            m = layer["mlp"]
            x = x + (gated_unit(h, w, p + "mlp.") if m["kind"] == "dense" else mixture(h, w, p + "mlp.", m))
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return (x @ w["head"].T) * config["logit_scale"]
