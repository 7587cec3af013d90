"""A plain, slow evaluation of the Pivinex decoder in float64, one function per mechanism, written from the
design's equations and sharing no code with the package.  A whole sequence at a time, no cache: every token's
keys and values are recomputed from the layer's input.

Weights are a dict name -> torch tensor (any dtype; widened here), the configuration is the dict that
``config.json`` holds.  ``lowp=True`` rounds to bfloat16 where an engine's bfloat16 path may (operands and results
of matrix products, the cached latent and key part, the queries, the heads' outputs, activations); norms, angles,
scores, the softmax, the router and the stream stay exact.  It measures what rounding alone costs.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def _r(x, lowp):
    return x.to(torch.bfloat16).to(F64) if lowp else x


def matmul(x, w, lowp=False):
    """x W^T for a weight stored [out, in]."""
    return _r(_r(x, lowp) @ w.to(F64).T, lowp)


def layer_norm(x, gain, eps):
    """(x - mean) / sqrt(var + eps) * gain over the last axis; var is the mean squared deviation; no bias."""
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    var = (dev * dev).mean(-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * gain


def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_pairs(v, positions, base, dims):
    """Rotation of neighbouring pairs: (v[2i], v[2i+1]) turns by the angle p * base^(-2i / dims) for i < dims / 2;
    entries from ``dims`` on stay.  ``v`` [T, ..., n], ``positions`` [T]."""
    out = v.clone()
    T = v.shape[0]
    for i in range(dims // 2):
        freq = float(base) ** (-2.0 * i / dims)
        ang = positions.to(F64) * freq
        shape = [T] + [1] * (v.dim() - 2)
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def latent_attention(h, w, prefix, mixer, eps, lowp=False):
    """Softmax attention whose keys and values are expanded per head from one low-rank latent per token and one
    rotated key part shared by the heads.  ``h`` [T, width] is one sequence from position 0; returns [T, width]."""
    T = h.shape[0]
    H, dn, dr, dv = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"]
    rank = mixer["kv_rank"]
    g = lambda n: w[prefix + n].to(F64)
    pos = torch.arange(T)
    cq = _r(rms_norm(matmul(h, g("dq"), lowp), g("dq.norm"), eps), lowp)
    q = matmul(cq, g("uq"), lowp).view(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], _r(rotate_pairs(q[..., dn:], pos, mixer["rot"]["base"], mixer["rot"]["dims"]), lowp)
    down = matmul(h, g("dkv"), lowp)
    c = _r(rms_norm(down[:, :rank], g("dkv.norm"), eps), lowp)
    k_rot = _r(rotate_pairs(down[:, rank:], pos, mixer["rot"]["base"], mixer["rot"]["dims"]), lowp)       # [T, dr], all heads
    k_plain = matmul(c, g("uk"), lowp).view(T, H, dn)
    val = matmul(c, g("uv"), lowp).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * mixer["scale"]
    i, j = pos.view(-1, 1), pos.view(1, -1)
    seen = (j <= i)
    size = (mixer.get("mask") or {}).get("size")
    if size:
        seen = seen & (i - j < size)
    scores = scores.masked_fill(~seen, float("-inf"))
    p = torch.softmax(scores, dim=-1)
    heads = _r(torch.einsum("hij,jhd->ihd", p, val).reshape(T, H * dv), lowp)
    return matmul(heads, g("o"), lowp)


def dense_ffn(h, w, prefix, lowp=False):
    g = lambda n: w[prefix + n].to(F64)
    return matmul(_r(gelu_tanh(matmul(h, g("gate"), lowp)) * matmul(h, g("up"), lowp), lowp), g("down"), lowp)


def route(h, w, prefix, router, margins=None):
    """Per token the chosen experts and their weights: scores are a softmax over all router outputs; the choice
    adds a correction per expert to the scores, the weights are the plain scores times a constant.  ``margins``
    receives, per token, by how much the last chosen output beat the best one left out."""
    z = h @ w[prefix + "router"].to(F64).T
    s = torch.softmax(z, dim=-1)
    choice = s + w[prefix + "correction"].to(F64)
    pick = choice.topk(router["top"], dim=-1).indices
    if margins is not None and router["top"] < choice.shape[-1]:
        ranked = choice.sort(dim=-1, descending=True).values
        margins.extend((ranked[..., router["top"] - 1] - ranked[..., router["top"]]).reshape(-1).tolist())
    return pick, s.gather(-1, pick) * router["scale"]


def moe_ffn(h, w, prefix, mlp, lowp=False, margins=None):
    router = mlp["router"]
    n_real = router["experts"]
    pick, weight = route(h, w, prefix, router, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(pick[t].tolist(), weight[t]):
            if e >= n_real:            # an expert without weights: the input itself
                out[t] += a * h[t]
                continue
            g = lambda n: w[f"{prefix}e{e}.{n}"].to(F64)
            out[t] += a * matmul(_r(silu(matmul(h[t], g("gate"), lowp)) * matmul(h[t], g("up"), lowp), lowp), g("down"), lowp)
    return out


def layer(x, w, i, cfg, lowp=False, margins=None):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    pre = f"l{i}."
    h = _r(layer_norm(x, w[pre + "norm1"].to(F64), eps), lowp)
    if L["type"] != "latent_attention":
        raise ValueError(L["type"])
    branch = latent_attention(h, w, pre + "mix.", L["mixer"], eps, lowp) * w[pre + "ls1"].to(F64)
    mlp = L.get("mlp")
    if mlp:
        f = dense_ffn(h, w, pre + "mlp.", lowp) if mlp["kind"] == "dense" else moe_ffn(h, w, pre + "mlp.", mlp, lowp, margins)
        branch = branch + f * w[pre + "ls2"].to(F64)
    return x + cfg["residual_mult"] * branch


def layer_order(cfg):
    """(layer index, first of a repeated pass?) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = [(i, False) for i in range(loop["start"])]
    for rep in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, rep > 0 and i == loop["start"]))
    order += [(i, False) for i in range(loop["stop"], n)]
    return order


def forward(tokens, w, cfg, streams=None, lowp=False, margins=None):
    """Logits [T, vocab] (float64) of one sequence; ``streams``: a list that receives the stream after every
    layer run; ``margins``: a list that receives every router decision's margin."""
    eps = cfg["norm"]["eps"]
    e = layer_norm(w["embed"].to(F64)[torch.as_tensor(tokens)], w["embed.norm"].to(F64), eps)
    x = e
    for i, again in layer_order(cfg):
        if again:
            x = x + e
        x = layer(x, w, i, cfg, lowp, margins)
        if streams is not None:
            streams.append(x)
    return _r(layer_norm(x, w["final.norm"].to(F64), eps), lowp) @ w["head"].to(F64).T
