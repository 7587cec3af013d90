"""The Pivinex decoder as data: an embedding with a layer norm behind it; layers in which the mixer and the
feed-forward both read ONE layer norm's output and enter the stream together, each with a gain per feature and all
times a constant; a span of layers that runs several times in a row with the same weights, every pass with a cache of
its own and the embedding's output fed in again before every pass but the first; a final layer norm and a head.

* mixer ``latent_attention``: softmax attention over a sliding window whose keys and values are maps of one cached
  low-rank latent per token, with queries that go through a latent of their own and a rotated part of neighbouring
  pairs beside the unrotated one.
* feed-forward: gated with the tanh form of gelu, or routed (gated silu experts, softmax router with a correction
  that only the choice sees, router outputs without weights that return their input), or none.

This file only turns the configuration into a ModelSpec, layer by layer; all the computing is in ``pyre_b200.parts``.
"""

from __future__ import annotations

from ..config.model_config import PivinexConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerCall, ModelSpec


def build_pivinex(cfg: PivinexConfig) -> ModelSpec:
    def norm():
        return PartSpec("layer_norm", {"width": cfg.width, "eps": cfg.norm_eps, "tensor_name": ""})

    blocks = []
    for L in cfg.layers:
        position = PartSpec("rotary", {"head_dim": L.rot_dim, "theta": L.rot_base, "rotary_dim": L.rot_dims,
                                       "pairing": "interleaved", "exact_frequencies": True})
        mixer = PartSpec("latent_attention", {
            "width": cfg.width, "n_heads": L.heads, "head_dim": L.dim, "rope_dim": L.rot_dim, "v_head_dim": L.vdim,
            "q_rank": L.q_rank, "kv_rank": L.kv_rank, "scale": L.scale, "eps": cfg.norm_eps, "window": L.window or None,
            "position": position})
        ffn = None
        if L.mlp_kind == "dense":
            ffn = PartSpec("gated_mlp", {"width": cfg.width, "intermediate": L.ff, "activation": "gelu_tanh",
                                         "names": {"gate": "gate", "up": "up", "down": "down"}, "weight_suffix": ""})
        elif L.mlp_kind == "moe":
            ffn = PartSpec("routed_mlp", {"width": cfg.width, "intermediate": L.ff, "n_experts": L.experts,
                                          "n_identity": L.identity, "top": L.top, "scale": L.router_scale,
                                          "activation": "silu", "correction": True})
        blocks.append(PartSpec("parallel", {
            "width": cfg.width, "norm1": norm(), "mixer": mixer, "ffn": ffn, "residual_mult": cfg.residual_mult,
            "layer_scale": True, "names": {"norm1": "norm1", "mixer": "mix.", "ffn": "mlp.", "ls1": "ls1", "ls2": "ls2"}}))
    # a layer of the repeated span appears once per pass; every appearance has a cache layer of its own
    schedule = [LayerCall(i, add_embedding=again) for i, again in cfg.layer_order()]
    return ModelSpec(
        embed=PartSpec("token_embedding", {"vocab": cfg.vocab, "width": cfg.width, "tensor_name": "", "norm": norm()}),
        blocks=blocks,
        final_norm=norm(),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width, "tensor_name": ""}),
        schedule=schedule,
        embed_prefix="embed", block_prefix="l{i}.", final_norm_prefix="final.norm", head_prefix="head",
        vocab_size=cfg.vocab,
        max_positions=0,
    )


register_architecture(PivinexConfig.architecture, PivinexConfig, build_pivinex)
