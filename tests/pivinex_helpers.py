"""Fixtures of the Pivinex tests: small configurations that differ in every size and option, model folders with
random weights, and the plain implementation's logits."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch
from safetensors.torch import load_file, save_file

from modovik_helpers import compare  # noqa: F401  (the same bounds: rounding of the plain model, no wider)
from plain import pivinex_plain


def _mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base=10000.0, rot_dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
            "mask": {"size": window}, "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}


def _layer(mixer, mlp=None):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, identity, top, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}


# A: a span in the middle that runs three times (layers 1-2), mixers of two shapes (so two cache groups), windows of
#    11 and 23 tokens on pages of 16, one layer without a feed-forward, a routed one with one weightless output.
PIV_A = {"architecture": "Pivinex", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
         "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
    _layer(_mixer(3, 16, 8, 24, 40, 24, 0.2, 11), _dense(160)),
    _layer(_mixer(4, 32, 16, 16, 48, 48, 0.15, 23), _moe(64, 5, 1, 2, 1.0)),
    _layer(_mixer(4, 32, 16, 16, 48, 48, 0.15, 23)),
    _layer(_mixer(3, 16, 8, 24, 40, 24, 0.2, 11), _moe(32, 4, 0, 1, 2.5)),
]}
# B: no size is a multiple of 8 (width 92, latents of 20 and 36, heads of 20 + 12 and values of 12: the library
#    product for odd K, the scalar paths, the exact attention kernel in both dtypes), only part of the rotated part
#    rotated, a window of 7 on pages of 8, no repeated span, as many chosen as there are experts with weights.
PIV_B = {"architecture": "Pivinex", "vocab": 333, "width": 92, "norm": {"eps": 3e-6}, "residual_mult": 1.0, "layers": [
    _layer(_mixer(5, 20, 12, 12, 20, 36, 0.18, 7, base=500.0, rot_dims=8), _moe(20, 3, 2, 3, 0.7)),
    _layer(_mixer(5, 20, 12, 12, 20, 36, 0.18, 7, base=500.0, rot_dims=8), _dense(66)),
    _layer(_mixer(2, 28, 4, 40, 12, 52, 0.3, 1000)),
]}
# C: sizes of the tensor-core paths: a latent of 192 (two column blocks of the attention kernel), eight heads, a window
#    of 64 on pages of 32, the whole model twice, dense feed-forwards wide enough for the gated product, eight experts.
PIV_C = {"architecture": "Pivinex", "vocab": 640, "width": 256, "norm": {"eps": 1e-6}, "residual_mult": 0.25,
         "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
    _layer(_mixer(8, 64, 32, 64, 96, 192, 0.09, 64, base=1000000.0), _dense(512)),
    _layer(_mixer(8, 64, 32, 64, 96, 192, 0.09, 64, base=1000000.0), _moe(128, 8, 0, 2, 1.0)),
]}
# D: more heads than a row tile of the attention kernel takes (72 > 64), a latent of 64 with a key part of 16, a query
#    latent of 36 (a stacked down-projection of 116 rows, no multiple of 8, on the tensor-core product; the queries'
#    up-projection with an inner size of 36 on the library product), a window far wider than any request, one layer.
PIV_D = {"architecture": "Pivinex", "vocab": 256, "width": 128, "norm": {"eps": 1e-5}, "residual_mult": 0.8, "layers": [
    _layer(_mixer(72, 16, 16, 8, 36, 64, 0.2, 100000), _dense(128)),
]}
PIV = {"A": PIV_A, "B": PIV_B, "C": PIV_C, "D": PIV_D}
PIV_PAGE_SIZE = {"A": 16, "B": 8, "C": 32, "D": 16}
ROUTER_MARGIN = 1.5e-3     # a router decision closer than this could fall either way under bfloat16 rounding (decisions
                           # that differed between the plain model and its bfloat16 emulation had margins below 4e-4)


def make_pivinex_dir(path: Path, raw: dict, seed: int, sharpen: float = 4.0, matrix_scale: float = 2.0) -> dict:
    """config.json + model.safetensors (fp32 values that bfloat16 holds exactly) from the package's random mode.
    The maps that make queries and keys are scaled up so that attention is peaked (with small random weights every
    score is near zero and a wrong key would change nothing), the router's so that its scores differ."""
    from pyre_b200.config import config_from_dict
    from pyre_b200.weights import random_state

    path.mkdir(parents=True, exist_ok=True)
    state = random_state(config_from_dict(raw), seed)
    for name in state:
        if name.endswith((".mix.uq", ".mix.dkv")):
            state[name] = state[name] * sharpen
        elif name.endswith(".mlp.router"):
            state[name] = state[name] * 6.0
        elif state[name].dim() == 2:
            state[name] = state[name] * matrix_scale
        state[name] = state[name].to(torch.bfloat16).to(torch.float32)
    (path / "config.json").write_text(json.dumps(raw))
    save_file({k: v.contiguous() for k, v in state.items()}, str(path / "model.safetensors"))
    return state


def decided_ids(path: Path, length: int, seed: int, chunk: int = 6) -> list:
    """Random token ids on which no router decision of the model is a close call: grown a few tokens at a time, a
    piece drawn again while any decision at its positions is closer than ROUTER_MARGIN (a decision depends on the
    tokens up to its own only).  A model without routers gets plain random ids."""
    raw = json.loads((Path(path) / "config.json").read_text())
    rng = np.random.default_rng(seed)
    if not any((L.get("mlp") or {}).get("kind") == "moe" for L in raw["layers"]):
        return [int(x) for x in rng.integers(0, raw["vocab"], length)]
    w = load_file(str(Path(path) / "model.safetensors"))
    ids: list = []
    while len(ids) < length:
        n = min(chunk, length - len(ids))
        for _ in range(200):
            piece = [int(x) for x in rng.integers(0, raw["vocab"], n)]
            margins: list = []
            with torch.inference_mode():
                pivinex_plain.forward(ids + piece, w, raw, margins=margins)
            T = len(ids) + n
            per_run = np.asarray(margins).reshape(-1, T)[:, -n:]       # one row per run of a routed layer that leaves outputs out
            if per_run.size == 0 or per_run.min() > ROUTER_MARGIN:
                break
        else:
            raise AssertionError("no piece of tokens gave decided router choices")
        ids += piece
    return ids


def plain_logits(path: Path, ids, lowp: bool = False) -> np.ndarray:
    raw = json.loads((Path(path) / "config.json").read_text())
    w = load_file(str(Path(path) / "model.safetensors"))
    with torch.inference_mode():
        return pivinex_plain.forward(list(ids), w, raw, lowp=lowp).numpy()
