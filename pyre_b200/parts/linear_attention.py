"""Linear attention with a constant decay per head: a mixer whose memory is a matrix of fixed size per request
and head, kept in a state slot of the cache manager instead of pages."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import Part, StateSpec, register_part


class DecayLinearAttention(Part):
    """Per head, with q_t, k_t of ``head_dim`` and v_t of ``v_head_dim`` entries (each act(W h), ``activation``
    silu or None):

        S_t = decay_h S_(t-1) + k_t v_t^T        o_t = S_t^T q_t        (no other scale)

    The state S [head_dim, v_head_dim] is fp32, starts at zero when a request begins and is carried from token
    to token in the request's state slot; the decays are constants of the model (``decay``, one per head).  The
    concatenated heads then pass an RMS norm over the whole row (plain weight, ``eps``; name ``norm``), are
    multiplied by sigmoid(W_g h) when ``out_gate`` and projected by W_o.  The recurrence, the norm and the gate are
    computed in fp32; the four projections are one product [q | k | v | gate].

    ``names``: the checkpoint's full local names of the tensors."""

    DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                     "o": "o_proj.weight", "norm": "norm.weight"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, n_heads: int, head_dim: int, v_head_dim: int, decay, eps: float,
                 activation: "str | None" = "silu", out_gate: bool = True, names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.n_heads, self.head_dim, self.v_head_dim = int(width), int(n_heads), int(head_dim), int(v_head_dim)
        decay = [float(d) for d in decay]
        if len(decay) != self.n_heads:
            raise ValueError(f"{len(decay)} decays for {self.n_heads} heads")
        if not 1 <= self.head_dim <= 256:
            raise ops.UnsupportedSize(f"linear attention takes query/key sizes up to 256, got {head_dim}")
        if activation not in (None, "silu"):
            raise ops.UnsupportedSize(f"linear attention: activation {activation!r} is not implemented")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(self.device)
        self.eps, self.activation, self.out_gate = float(eps), activation, bool(out_gate)
        qk, vv = self.n_heads * self.head_dim, self.n_heads * self.v_head_dim
        self.q_col, self.k_col, self.v_col, self.g_col = 0, qk, 2 * qk, 2 * qk + vv
        self.w_proj = self.w_o = self.norm_w = None

    def tensors(self):
        n = self.names
        qk, vv = self.n_heads * self.head_dim, self.n_heads * self.v_head_dim
        t = {n["q"]: TensorSpec((qk, self.width)), n["k"]: TensorSpec((qk, self.width)), n["v"]: TensorSpec((vv, self.width))}
        if self.out_gate:
            t[n["g"]] = TensorSpec((vv, self.width))
        t[n["o"]] = TensorSpec((self.width, vv))
        t[n["norm"]] = TensorSpec((vv,), role="vector", init=("normal", 1.0, 0.1))
        return t

    def load(self, tensors):
        n = self.names
        stack = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]] + ([tensors[n["g"]]] if self.out_gate else [])
        self.w_proj = torch.cat(stack, dim=0).contiguous()
        self.w_o, self.norm_w = tensors[n["o"]], tensors[n["norm"]]

    def kernel_libraries(self):
        return ["blockops", "linear_attention", "elementwise"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def cache_spec(self):
        return None

    def state_spec(self):
        return StateSpec((self.n_heads, self.head_dim, self.v_head_dim), torch.float32)

    def forward(self, ctx, h, call):
        st = ctx.state_group(call.state_group)
        with lib.section("qkv"):
            proj = ops.materialize(ops.linear(h, self.w_proj))
        o = ops.linear_attention(proj, self.q_col, self.k_col, self.v_col, st.buffer[call.state_layer], st.slots,
                                 ctx.cu_seqlens, self.decay, self.n_heads, self.head_dim, self.v_head_dim, self.activation,
                                 lens=ctx.cu_seqlens_host[1:] - ctx.cu_seqlens_host[:-1])
        a = ops.rmsnorm_gate(o, self.norm_w, self.eps, proj if self.out_gate else None, self.g_col, self.dtype)
        with lib.section("o"):
            return ops.linear(a, self.w_o, partials_ok=True)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
