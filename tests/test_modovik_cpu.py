"""Modovik on the host side: the configuration, the registry, the model as data, and (with plain torch stand-ins
for the kernels) the package's own parts, cache manager, step function and replay loop against the plain
implementation, under cutting, batching and reuse of pages and state slots."""

import json

import numpy as np
import pytest
import torch

import helpers as H
import modovik_helpers as MH
import standins
from pyre_b200.config import ConfigError, ModovikConfig, config_from_dict
from pyre_b200.config.registry import architecture_of
from pyre_b200.models.model import Model, tensor_table


def test_config_round_trip_and_registry():
    for raw in MH.MODO.values():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, ModovikConfig)
        assert config_from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    cfg = config_from_dict(MH.MODO_P)
    assert [L.kind for L in cfg.layers] == ["lightning", "attention", "lightning", "attention"]
    assert cfg.layers[3].kv_from == 1 and cfg.layers[1].kv_from == -1 and cfg.layers[2].ff == 0 and cfg.layers[0].ff == 160


@pytest.mark.parametrize("edit, word", [
    (lambda r: r["layers"][1].update(type="conv"), "type"),
    (lambda r: r["layers"][1]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=40), "rot.dims"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(dim=16), "layer 1"),
    (lambda r: r["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda r: r["layers"][0]["mlp"].update(kind="routed"), "dense"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["layers"][1]["mixer"].pop("scale"), "scale"),
])
def test_config_errors_name_the_key(edit, word):
    raw = json.loads(json.dumps(MH.MODO_P))
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_tensor_names_and_cache_groups():
    cfg = config_from_dict(MH.MODO_P)
    spec = architecture_of(cfg).build(cfg)
    table = tensor_table(spec)
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.norm", "l0.mlp.up", "l1.mix.q.norm",
            "l1.mix.k.norm", "l1.mix.g", "l3.mix.q", "l3.mix.q.norm", "l3.mlp.down"} <= set(table)
    assert "l3.mix.k" not in table and "l3.mix.v" not in table and "l3.mix.k.norm" not in table
    assert "l1.norm2" not in table and "l2.mlp.up" not in table
    assert table["l1.mix.v"].shape == (2 * 16, 96) and table["l1.mix.g"].shape == (6 * 16, 96)
    assert table["l0.mix.v"].shape == (3 * 24, 96) and table["l2.mix.norm"].shape == (2 * 40,)
    model = Model(spec, torch.float32, "cpu")
    # both attention layers share one cache layer: the reader writes nothing
    assert len(model.kv_groups) == 1 and model.kv_groups[0].n_layers == 1 and model.kv_groups[0].spec.head_dim == 32
    assert [c.kv_write for c in model.calls if c.kv_group is not None] == [True, False]
    # two recurrent layers with states of different shapes: two state groups
    assert [g.spec.shape for g in model.state_groups] == [(3, 16, 24), (2, 24, 40)]
    assert "linear_attention" in model.kernel_libraries() and "blockops" in model.kernel_libraries()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for n, name in enumerate(["P", "R"]):
        d = tmp_path_factory.mktemp(f"modo_{name}")
        MH.make_modovik_dir(d, MH.MODO[name], seed=300 + n)
        reqs = {f"{name}{i}": H.random_ids(MH.MODO[name]["vocab"], L, seed=17 * n + i) for i, L in enumerate([1, 2, 19, 37, 50])}
        out[name] = (d, reqs, {rid: MH.plain_logits(d, ids) for rid, ids in reqs.items()})
    return out


def _replay_on_cpu(monkeypatch, folder, steps, page_size, max_requests=4):
    import tempfile
    from pathlib import Path
    from pyre_b200.engine import replay as rp
    from pyre_b200.models.model import load_model

    standins.install(monkeypatch)
    model, _cfg = load_model(folder, "cpu", "float32")
    cache, stepper = rp.runtime_for_model(model, H.max_live_tokens(steps), page_size, max_requests, poison=True, cuda_graphs=False)
    with tempfile.TemporaryDirectory() as out:
        rp.replay(stepper, [json.dumps(s) for s in steps], Path(out), done=lambda m: None)
        got = H.collect_trace_logits(steps, lambda n: np.fromfile(Path(out) / f"{n}.f32", dtype="<f4").reshape(-1, model.vocab_size))
    cache.check()
    assert not cache.live() and cache.state.num_free == max_requests
    return got


@pytest.mark.parametrize("name", ["P", "R"])
def test_host_side_portions_and_mixed_batches(monkeypatch, folders, name):
    d, reqs, plain = folders[name]
    steps = []
    for k, (rid, ids) in enumerate(reqs.items()):
        steps += H.trace_portions(rid, ids, [[2, 9, 3], [5, 2, 16]][k % 2], first_step=len(steps))
    MH.compare(_replay_on_cpu(monkeypatch, d, steps, MH.MODO_PAGE_SIZE[name]), plain, "float32", "portions")
    many = {f"{rid}r{rep}": ids for rep in range(2) for rid, ids in reqs.items()}     # ten requests through four slots
    steps = H.trace_mixed(many, seed=5, max_live=4)
    got = _replay_on_cpu(monkeypatch, d, steps, MH.MODO_PAGE_SIZE[name])
    MH.compare(got, {f"{rid}r{rep}": plain[rid] for rep in range(2) for rid in reqs}, "float32", "mixed")


def test_random_model_folder_loads(tmp_path, monkeypatch):
    from pyre_b200.models.model import load_model
    from pyre_b200.weights import write_random_model

    standins.install(monkeypatch)
    cfg = config_from_dict(MH.MODO_Q)
    write_random_model(tmp_path, cfg, seed=1)
    assert json.loads((tmp_path / "config.json").read_text())["architecture"] == "Modovik"
    model, loaded = load_model(tmp_path, "cpu", "float32")
    assert loaded == cfg and model.loaded
