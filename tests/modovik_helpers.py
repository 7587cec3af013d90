"""Fixtures of the Modovik tests: small configurations that differ in every size and option, model folders
with random weights, and the plain implementation's logits."""

from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch
from safetensors.torch import load_file, save_file

from plain import modovik_plain


def _attn(heads, kv_heads, dim, vdim, rot_dims, base, scale, kv_from=None, ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
             "rot": {"dims": rot_dims, "base": base}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _lightning(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


# P: a recurrent layer first (with a feed-forward), attention without one, a reader of another layer's cache two
#    layers on, heads of 32 / 16 (cache rows of 32), three query heads per key/value head.
MODO_P = {"architecture": "Modovik", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "layers": [
    _lightning(3, 16, 24, [0.5, 0.9, 0.99], ff=160),
    _attn(6, 2, 32, 16, 8, 10000.0, 0.3),
    _lightning(2, 24, 40, [1.0, 0.8]),
    _attn(6, 2, 32, 16, 8, 10000.0, 0.3, kv_from=1, ff=64),
]}
# Q: key and value sizes equal, the whole head rotated, one key/value head, cache rows of 64; the recurrent layer last.
MODO_Q = {"architecture": "Modovik", "vocab": 512, "width": 128, "norm": {"eps": 1e-5}, "layers": [
    _attn(4, 1, 64, 64, 64, 500000.0, 0.125, ff=256),
    _attn(4, 1, 64, 64, 64, 500000.0, 0.125, kv_from=0),
    _lightning(4, 64, 32, [0.7, 0.95, 0.999, 0.9999], ff=128),
]}
# R: no size is a multiple of 8: a width of 92, heads of 24 / 40 (cache rows of 48 in float32, 64 in bfloat16), no
#    rotation at all, as many key/value heads as query heads, an odd vocabulary.
MODO_R = {"architecture": "Modovik", "vocab": 333, "width": 92, "norm": {"eps": 3e-6}, "layers": [
    _attn(5, 5, 24, 40, 0, 10000.0, 0.2, ff=66),
    _lightning(5, 20, 12, [0.3, 0.6, 0.9, 0.97, 0.995]),
    _attn(5, 5, 24, 40, 0, 10000.0, 0.2),
]}
# S: large heads: 80 / 112 (cache rows of 128) and 144 / 64 (rows of 144: the exact kernel in both dtypes); a
#    recurrent layer with 256 query/key dims.
MODO_S = {"architecture": "Modovik", "vocab": 640, "width": 256, "norm": {"eps": 1e-5}, "layers": [
    _attn(4, 2, 80, 112, 32, 1000000.0, 0.11, ff=384),
    _lightning(2, 256, 48, [0.98, 0.9995]),
    _attn(2, 1, 144, 64, 16, 10000.0, 0.083, ff=128),
    _attn(4, 2, 80, 112, 32, 1000000.0, 0.11, kv_from=0),
]}
MODO = {"P": MODO_P, "Q": MODO_Q, "R": MODO_R, "S": MODO_S}
MODO_PAGE_SIZE = {"P": 16, "Q": 8, "R": 32, "S": 16}


def make_modovik_dir(path: Path, raw: dict, seed: int, sharpen: float = 5.0, matrix_scale: float = 2.0) -> dict:
    """config.json + model.safetensors (fp32 values that bfloat16 holds exactly, as a checkpoint of this design
    stores them) from the package's random mode; the query and key projections are scaled up so that attention
    is peaked: with small random weights every score is near zero and a wrong key would change nothing."""
    from pyre_b200.config import config_from_dict
    from pyre_b200.weights import random_state

    path.mkdir(parents=True, exist_ok=True)
    state = random_state(config_from_dict(raw), seed)
    for name in state:
        if name.endswith((".mix.q", ".mix.k")):
            state[name] = state[name] * sharpen
        elif state[name].dim() == 2:
            state[name] = state[name] * matrix_scale
        state[name] = state[name].to(torch.bfloat16).to(torch.float32)
    (path / "config.json").write_text(json.dumps(raw))
    save_file({k: v.contiguous() for k, v in state.items()}, str(path / "model.safetensors"))
    return state


def plain_logits(path: Path, ids, lowp: bool = False) -> np.ndarray:
    raw = json.loads((Path(path) / "config.json").read_text())
    w = load_file(str(Path(path) / "model.safetensors"))
    with torch.inference_mode():
        return modovik_plain.forward(list(ids), w, raw, lowp=lowp).numpy()


def compare(got: dict, want: dict, dtype: str, what: str, lowp_rms: float = 0.0):
    """float32: every logit within rounding of the plain implementation.  bfloat16: the engine's rms error against
    the plain implementation is at most twice that of the plain implementation rounded to bfloat16 where the
    engine may round, and no logit is off by more than sixteen times that rms (a wrong key, page, slot or position
    moves logits by their whole spread)."""
    assert set(got) == set(want), f"{what}: requests differ"
    sq, cnt = 0.0, 0
    for rid in want:
        g, w = got[rid], want[rid]
        assert g.shape == w.shape, f"{what} {rid}: shape {g.shape} != {w.shape}"
        assert np.isfinite(g).all(), f"{what} {rid}: non-finite logits at rows {np.unique(np.where(~np.isfinite(g))[0])[:8]}"
        err = np.abs(g - w)
        bound = 3e-5 + 2e-4 * np.abs(w) if dtype == "float32" else np.full_like(w, 16.0 * lowp_rms)
        sq, cnt = sq + float((err.astype(np.float64) ** 2).sum()), cnt + err.size
        bad = err > bound
        if bad.any():
            row = int(np.where(bad.any(axis=1))[0][0])
            raise AssertionError(f"{what} {rid} ({dtype}): first wrong token at position {row} of {g.shape[0]}; "
                                 f"max |diff| there {err[row].max():.3e}, bound {bound[row].max():.3e}, "
                                 f"overall max {err.max():.3e}, logits std {w.std():.3f}")
    if dtype == "bfloat16":
        rms = math.sqrt(sq / cnt)
        assert rms <= 2.0 * lowp_rms, f"{what} (bfloat16): rms error {rms:.3e} against {lowp_rms:.3e} of plain rounding"
