"""A plain, slow implementation of the Modovik decoder, one function per mechanism, in float64 torch on the CPU.

It is the oracle of the tests: written from the design's equations, it shares no code with ``pyre_b200``.
A whole sequence is evaluated at once from position 0 with no cache and no state carried over; the engine has to
give the same logits however it cuts, batches and caches.

``lowp=True`` rounds to bfloat16 where the engine's bfloat16 path may (inputs and results of matrix products,
results of activations, what the cache stores); everything the design wants in 32-bit stays unrounded.  The
difference between the two runs is the yardstick for the engine's rounding error.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def _r(x: torch.Tensor, lowp: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(F) if lowp else x


def matmul(x, w, lowp=False):
    """y = x W^T for a weight stored [out, in]."""
    return _r(_r(x, lowp) @ w.to(F).t(), lowp)


def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def rotate_leading(x, positions, dims, base):
    """x [T, heads, d]: dimension i < dims/2 of every head is paired with dimension i + dims/2; the pair (u, v) at
    position p turns by the angle p * base^(-2 i / dims).  Dimensions from ``dims`` on are left alone."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sink_attention(q, k, v, scale, sink=0.0):
    """Causal attention of q [T, H, d] over k [T, G, d], v [T, G, dv] (query head h uses key/value head
    h // (H / G)) whose softmax has one more term exp(sink) in the denominator and no value for it."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, h]) * scale
            top = max(float(s.max()), sink)
            e = torch.exp(s - top)
            out[t, h] = (e / (e.sum() + math.exp(sink - top))) @ v[:t + 1, g]
    return out


def decayed_linear_attention(q, k, v, decay):
    """Per head: S_t = decay_h S_(t-1) + k_t v_t^T from S = 0, o_t = S_t^T q_t.  q, k [T, H, d], v [T, H, dv]."""
    T, H, d = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        S = torch.zeros(d, v.shape[2], dtype=F)
        for t in range(T):
            S = float(decay[h]) * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.t() @ q[t, h]
    return out


def attention_mixer(h, w, p, m, eps, positions, shared_kv, lowp):
    """The softmax mixer of one layer; returns (output [T, width], (keys, values) as cached)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = matmul(h, w[p + "q"], lowp).reshape(T, H, d)
    q = _r(rotate_leading(rms_norm(q, w[p + "q.norm"].to(F), eps), positions, rot["dims"], rot["base"]), lowp)
    if shared_kv is None:
        k = matmul(h, w[p + "k"], lowp).reshape(T, G, d)
        k = _r(rotate_leading(rms_norm(k, w[p + "k.norm"].to(F), eps), positions, rot["dims"], rot["base"]), lowp)
        v = matmul(h, w[p + "v"], lowp).reshape(T, G, dv)
    else:
        k, v = shared_kv
    a = _r(sink_attention(q, k, v, m["scale"], 0.0), lowp).reshape(T, H * dv)
    a = _r(a * sigmoid(matmul(h, w[p + "g"], lowp)), lowp)
    return matmul(a, w[p + "o"], lowp), (k, v)


def lightning_mixer(h, w, p, m, eps, lowp):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(matmul(h, w[p + "q"], lowp)).reshape(T, H, d)
    k = silu(matmul(h, w[p + "k"], lowp)).reshape(T, H, d)
    v = silu(matmul(h, w[p + "v"], lowp)).reshape(T, H, dv)
    o = decayed_linear_attention(q, k, v, m["decay"]).reshape(T, H * dv)
    o = _r(rms_norm(o, w[p + "norm"].to(F), eps) * sigmoid(matmul(h, w[p + "g"], lowp)), lowp)
    return matmul(o, w[p + "o"], lowp)


def dense_ff(h, w, p, lowp):
    return matmul(_r(gelu_tanh(matmul(h, w[p + "up"], lowp)), lowp), w[p + "down"], lowp)


def forward(ids, w, raw, lowp=False, layers_out=None):
    """Logits [T, vocab] (float64) of the token ids of one sequence."""
    eps = raw["norm"]["eps"]
    T = len(ids)
    positions = torch.arange(T)
    x = w["embed"].to(F)[torch.tensor(list(ids), dtype=torch.long)]
    cached = {}
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "lightning":
            y = lightning_mixer(x, w, p, m, eps, lowp)
        else:
            src = m.get("kv_from")
            y, kv = attention_mixer(x, w, p, m, eps, positions, cached[src] if src is not None else None, lowp)
            if src is None:
                cached[i] = kv
        x = x + rms_norm(y, 1.0 + w[f"l{i}.norm1"].to(F), eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(dense_ff(x, w, f"l{i}.mlp.", lowp), 1.0 + w[f"l{i}.norm2"].to(F), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, 1.0 + w["final.norm"].to(F), eps)
    return _r(x, lowp) @ w["head"].to(F).t()
