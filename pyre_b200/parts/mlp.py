"""Dense feed-forwards: the gated one (SwiGLU, pyre/model.py:128-139) and the plain one (up, activation, down)."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import Part, register_part


class GatedMLP(Part):
    """down(act(gate(h)) * up(h)) without biases.  The gate and up weights are stacked
    into one [2 I, width] matrix at load, so one product feeds the activation; in bfloat16,
    when I is a multiple of 128, their rows alternate in blocks of 64 features so that one
    output tile of the product holds both halves and the activation runs in its epilogue.
    ``names``: the checkpoint's names of the three projections (default gate_proj, up_proj, down_proj);
    ``weight_suffix``: what follows a projection's name (".weight").  ``activation``: ``silu``, or ``gelu_tanh``
    (product, then the activation kernel on the stacked [gates | ups])."""

    DEFAULT_NAMES = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}

    graph_safe = True
    takes_scaled_rows = True      # ``h`` may be ``ops.ScaledRows``: the gate/up product applies the norm's 1/rms itself

    def __init__(self, dtype, device, width: int, intermediate: int, activation: str = "silu",
                 names: "dict[str, str] | None" = None, weight_suffix: str = ".weight"):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.suffix = str(weight_suffix)
        self.width, self.intermediate = int(width), int(intermediate)
        if activation not in ops.ACTIVATIONS:
            raise ops.UnsupportedSize(f"activation {activation!r}: implemented are {sorted(ops.ACTIVATIONS)}")
        self.activation = activation
        self.w_gate_up = self.w_down = None
        # the product's epilogue knows silu; another activation runs after the product on [gates | ups]
        self.interleaved = activation == "silu" and dtype == torch.bfloat16 and self.intermediate % (2 * ops.GATED_BLOCK) == 0
        if activation != "silu":
            self.takes_scaled_rows = False

    def tensors(self):
        n, sfx = self.names, self.suffix
        return {
            n["gate"] + sfx: TensorSpec((self.intermediate, self.width)),
            n["up"] + sfx: TensorSpec((self.intermediate, self.width)),
            n["down"] + sfx: TensorSpec((self.width, self.intermediate)),
        }

    def load(self, tensors):
        n, sfx = self.names, self.suffix
        gate, up = tensors[n["gate"] + sfx], tensors[n["up"] + sfx]
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[n["down"] + sfx]

    def kernel_libraries(self):
        return ["elementwise"] + (["parallel_block"] if self.activation != "silu" else []) + \
            (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def forward(self, ctx, h):
        with lib.section("gate_up"):
            if self.activation == "silu":
                act = ops.gated_linear(h, self.w_gate_up, self.interleaved)
            else:
                act = ops.act_mul(ops.materialize(ops.linear(h, self.w_gate_up)), self.activation)
        with lib.section("down"):
            return ops.linear(act, self.w_down, partials_ok=True, deferred_ok="residual")


register_part("ffn", "gated_mlp", GatedMLP)


class DenseMLP(Part):
    """down(act(up(h))) without biases: a feed-forward with one product before the activation.
    ``activation``: ``gelu_tanh`` (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))) or ``silu``, computed in fp32
    on the product's result.  ``names``: the checkpoint's full local names of the two weights."""

    DEFAULT_NAMES = {"up": "up_proj.weight", "down": "down_proj.weight"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, intermediate: int, activation: str = "gelu_tanh",
                 names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.intermediate = int(width), int(intermediate)
        if activation not in ops.ACTIVATIONS:
            raise ops.UnsupportedSize(f"activation {activation!r}: implemented are {sorted(ops.ACTIVATIONS)}")
        self.activation = activation
        self.w_up = self.w_down = None

    def tensors(self):
        return {self.names["up"]: TensorSpec((self.intermediate, self.width)),
                self.names["down"]: TensorSpec((self.width, self.intermediate))}

    def load(self, tensors):
        self.w_up, self.w_down = tensors[self.names["up"]], tensors[self.names["down"]]

    def kernel_libraries(self):
        return ["blockops", "elementwise"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def forward(self, ctx, h):
        with lib.section("up"):
            a = ops.linear_act(h, self.w_up, self.activation)
        with lib.section("down"):
            return ops.linear(a, self.w_down, partials_ok=True)


register_part("ffn", "dense_mlp", DenseMLP)


class RoutedMLP(Part):
    """A routed feed-forward: ``n_experts`` small gated feed-forwards (down(act(gate(h)) * up(h)), no biases) and
    ``n_identity`` further router outputs without weights whose "expert" returns h itself; each token uses ``top``
    of them.  The router's logits W_r h are fp32, the scores a softmax over ALL router outputs; the choice takes
    the ``top`` largest of score + correction (a tensor per router output, ``correction=True``), the weights are the
    chosen outputs' plain scores times ``scale``, not renormalised.  The result is the weighted sum.

    On the device throughout (no host reads): the router kernel, a sort of the (token, choice) pairs by expert,
    two products with one weight matrix per expert over the sorted pairs with the activation between them, and the
    weighted sum per token in fp32.  ``names``: the prefix of expert e's tensors (``expert``, formatted with e), the
    local names of its three projections, the router's and the correction's names."""

    DEFAULT_NAMES = {"expert": "e{e}.", "gate": "gate", "up": "up", "down": "down", "router": "router", "correction": "correction"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, intermediate: int, n_experts: int, top: int, scale: float = 1.0,
                 n_identity: int = 0, activation: str = "silu", correction: bool = True, names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.intermediate = int(width), int(intermediate)
        self.n_experts, self.n_identity, self.top, self.scale = int(n_experts), int(n_identity), int(top), float(scale)
        if activation not in ops.ACTIVATIONS:
            raise ops.UnsupportedSize(f"activation {activation!r}: implemented are {sorted(ops.ACTIVATIONS)}")
        if self.n_experts <= 0 or self.n_identity < 0 or not 0 < self.top <= self.n_experts + self.n_identity:
            raise ValueError(f"a routed feed-forward of {n_experts} + {n_identity} experts cannot choose {top}")
        self.activation, self.has_correction = activation, bool(correction)
        self.w_gate_up = self.w_down = self.w_router = self.correction = None

    def tensors(self):
        n, t = self.names, {}
        for e in range(self.n_experts):
            pre = n["expert"].format(e=e)
            t[pre + n["gate"]] = TensorSpec((self.intermediate, self.width))
            t[pre + n["up"]] = TensorSpec((self.intermediate, self.width))
            t[pre + n["down"]] = TensorSpec((self.width, self.intermediate))
        outs = self.n_experts + self.n_identity
        t[n["router"]] = TensorSpec((outs, self.width), role="vector", init=("normal", 0.0, 0.05))
        if self.has_correction:
            t[n["correction"]] = TensorSpec((outs,), role="vector", init=("normal", 0.0, 0.02))
        return t

    def load(self, tensors):
        n = self.names
        pres = [n["expert"].format(e=e) for e in range(self.n_experts)]
        self.w_gate_up = torch.stack([torch.cat([tensors[p + n["gate"]], tensors[p + n["up"]]], dim=0) for p in pres]).contiguous()
        self.w_down = torch.stack([tensors[p + n["down"]] for p in pres]).contiguous()
        self.w_router = tensors[n["router"]]
        self.correction = tensors[n["correction"]] if self.has_correction else None

    def kernel_libraries(self):
        return ["grouped", "parallel_block"]

    def forward(self, ctx, h):
        h = ops.materialize(h)
        T = h.shape[0]
        idx, weight = ops.route(h, self.w_router, self.correction, self.top, self.scale)
        offsets, place_of, src = ops.group_pairs(idx, self.n_experts)
        places = T * self.top
        with lib.section("experts_gate_up"):
            gu = ops.expert_linear(h, self.w_gate_up, offsets, src, places)
        act = ops.act_mul(gu, self.activation)
        with lib.section("experts_down"):
            y = ops.expert_linear(act, self.w_down, offsets, None, places, out_dtype=torch.float32)
        out = ops.combine_pairs(y, h, place_of, weight)
        # fp32 [T, width]: in bfloat16 it travels as the one part of a split product, which every norm adds unrounded
        return out if self.dtype == torch.float32 else ops.PartialSums(out.unsqueeze(0), self.dtype)


register_part("ffn", "routed_mlp", RoutedMLP)
