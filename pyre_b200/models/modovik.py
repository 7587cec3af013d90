"""The Modovik decoder as data: layers whose norms sit on the branches' outputs (x += norm(mixer(x)),
x += norm(ff(x)), each norm with a gain stored around zero), two kinds of mixer in any order, a dense feed-forward
with the tanh form of gelu (or none), a final norm and a head.

* ``attention``: grouped-query softmax attention with a value-less sink of score 0, an RMS norm per head on
  queries and keys, a rotation of the leading dims of each head, value heads of their own size, an output gate;
  a layer may read the keys and values that an earlier layer cached instead of projecting its own.
* ``lightning``: linear attention with a constant decay per head over a state of fixed size.

This file only turns the configuration into a ModelSpec, layer by layer; all the computing is in
``pyre_b200.parts``.
"""

from __future__ import annotations

from ..config.model_config import ModovikConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerCall, ModelSpec

SINK_SCORE = 0.0      # the sink's score: one is added to every softmax denominator


def build_modovik(cfg: ModovikConfig) -> ModelSpec:
    def norm():
        # the checkpoint stores gain - 1
        return PartSpec("rms_norm", {"width": cfg.width, "eps": cfg.norm_eps, "offset": 1.0, "tensor_name": ""})

    blocks, schedule = [], []
    for i, L in enumerate(cfg.layers):
        if L.kind == "lightning":
            mixer = PartSpec("decay_linear_attention", {
                "width": cfg.width, "n_heads": L.heads, "head_dim": L.dim, "v_head_dim": L.vdim, "decay": tuple(L.decay),
                "eps": cfg.norm_eps, "activation": "silu", "out_gate": True,
                "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}})
            schedule.append(LayerCall(i))
        else:
            position = PartSpec("rotary", {"head_dim": L.dim, "theta": L.rot_base, "rotary_dim": L.rot_dims,
                                           "exact_frequencies": True}) if L.rot_dims else PartSpec("none")
            shares = L.kv_from >= 0
            mixer = PartSpec("attention", {
                "width": cfg.width, "n_heads": L.heads, "n_kv_heads": L.kv_heads, "head_dim": L.dim, "v_head_dim": L.vdim,
                "qkv_bias": False, "o_bias": False, "scale": L.scale, "window": None, "position": position,
                "qk_norm": {"eps": cfg.norm_eps}, "sink": SINK_SCORE, "out_gate": True, "own_kv": not shares,
                "weight_suffix": "", "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "q_norm": "q.norm",
                                               "k_norm": "k.norm"}})
            schedule.append(LayerCall(i, cache=("layer", L.kv_from if shares else i), write=not shares))
        params = {"norm1": norm(), "mixer": mixer, "names": {"norm1": "norm1", "mixer": "mix.", "norm2": "norm2", "ffn": "mlp."}}
        if L.ff:
            params["norm2"] = norm()
            params["ffn"] = PartSpec("dense_mlp", {"width": cfg.width, "intermediate": L.ff, "activation": "gelu_tanh",
                                                   "names": {"up": "up", "down": "down"}})
        blocks.append(PartSpec("output_norm", params))
    return ModelSpec(
        embed=PartSpec("token_embedding", {"vocab": cfg.vocab, "width": cfg.width, "tensor_name": ""}),
        blocks=blocks,
        final_norm=norm(),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width, "tensor_name": ""}),
        schedule=schedule,
        embed_prefix="embed", block_prefix="l{i}.", final_norm_prefix="final.norm", head_prefix="head",
        vocab_size=cfg.vocab,
        max_positions=0,
    )


register_architecture(ModovikConfig.architecture, ModovikConfig, build_modovik)
