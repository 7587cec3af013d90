"""Pivinex on the host side: the configuration, the registry, the model as data, and (with plain torch stand-ins
for the kernels) the package's own parts, cache manager, step function and replay loop against the plain
implementation, under cutting, batching and reuse of pages."""

import json

import numpy as np
import pytest
import torch

import helpers as H
import pivinex_helpers as PH
import standins
from pyre_b200.config import ConfigError, config_from_dict
from pyre_b200.config.model_config import PivinexConfig
from pyre_b200.config.registry import architecture_of
from pyre_b200.models.model import Model, tensor_table


def test_config_round_trip_and_registry():
    for raw in PH.PIV.values():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, PivinexConfig)
        assert config_from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    cfg = config_from_dict(PH.PIV_A)
    assert [L.mlp_kind for L in cfg.layers] == ["dense", "moe", "", "moe"]
    assert (cfg.layers[1].experts, cfg.layers[1].identity, cfg.layers[1].top, cfg.layers[3].router_scale) == (5, 1, 2, 2.5)
    assert cfg.layer_order() == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert config_from_dict(PH.PIV_B).layer_order() == [(0, False), (1, False), (2, False)]
    assert config_from_dict(PH.PIV_B).layers[0].rot_dims == 8 and config_from_dict(PH.PIV_B).layers[0].rot_dim == 12


@pytest.mark.parametrize("edit, word", [
    (lambda r: r["layers"][1].update(type="conv"), "type"),
    (lambda r: r["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda r: r["layers"][0]["mlp"].update(kind="conv"), "kind"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["layers"][1]["mixer"].pop("scale"), "scale"),
])
def test_config_errors_name_the_key(edit, word):
    raw = json.loads(json.dumps(PH.PIV_A))
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_tensor_names_and_cache_groups():
    cfg = config_from_dict(PH.PIV_A)
    spec = architecture_of(cfg).build(cfg)
    table = tensor_table(spec)
    assert {"embed", "embed.norm", "head", "final.norm", "l0.norm1", "l0.ls1", "l0.ls2", "l0.mix.dq", "l0.mix.dq.norm",
            "l0.mix.dkv.norm", "l0.mlp.gate", "l1.mlp.e4.down", "l1.mlp.router", "l1.mlp.correction", "l2.ls1", "l3.mlp.e3.up"} <= set(table)
    assert table["l2.ls2"].optional and not table["l1.ls2"].optional and "l2.mlp.gate" not in table and "l1.mlp.e5.gate" not in table and "l0.norm2" not in table
    assert table["l1.mlp.router"].shape == (6, 96) and table["l3.mlp.correction"].shape == (4,)
    assert table["l0.mix.dkv"].shape == (24 + 8, 96) and table["l0.mix.uq"].shape == (3 * (16 + 8), 40)
    assert table["l1.mix.uk"].shape == (4 * 32, 48) and table["l1.mix.uv"].shape == (4 * 16, 48)
    model = Model(spec, torch.float32, "cpu")
    # eight entries of the schedule, each with a cache layer of its own; two shapes of mixer, two groups; one plane
    assert len(model.calls) == 8 and [c.block for c in model.calls] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [c.add_embedding for c in model.calls] == [False, False, False, True, False, True, False, False]
    assert sorted((g.spec.head_dim, g.spec.window, g.spec.planes, g.n_layers) for g in model.kv_groups) == [(32, 11, 1, 2), (64, 23, 1, 6)]
    assert not model.state_groups
    assert {"latent_attention", "grouped", "parallel_block"} <= set(model.kernel_libraries())


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for n, name in enumerate(["A", "B"]):
        d = tmp_path_factory.mktemp(f"piv_{name}")
        PH.make_pivinex_dir(d, PH.PIV[name], seed=300 + n)
        reqs = {f"{name}{i}": H.random_ids(PH.PIV[name]["vocab"], L, seed=17 * n + i) for i, L in enumerate([1, 2, 19, 37, 50])}
        out[name] = (d, reqs, {rid: PH.plain_logits(d, ids) for rid, ids in reqs.items()})
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


@pytest.mark.parametrize("name", ["A", "B"])
def test_host_side_portions_and_mixed_batches(monkeypatch, folders, name):
    d, reqs, plain = folders[name]
    steps = []
    for k, (rid, ids) in enumerate(reqs.items()):
        steps += H.trace_portions(rid, ids, [[2, 9, 3], [5, 2, 16]][k % 2], first_step=len(steps))
    PH.compare(_replay_on_cpu(monkeypatch, d, steps, PH.PIV_PAGE_SIZE[name]), plain, "float32", "portions")
    many = {f"{rid}r{rep}": ids for rep in range(2) for rid, ids in reqs.items()}     # ten requests, four alive at a time
    steps = H.trace_mixed(many, seed=5, max_live=4)
    got = _replay_on_cpu(monkeypatch, d, steps, PH.PIV_PAGE_SIZE[name])
    PH.compare(got, {f"{rid}r{rep}": plain[rid] for rep in range(2) for rid in reqs}, "float32", "mixed")


def test_a_window_gives_its_pages_back(monkeypatch, folders):
    """A request longer than its windows holds only the windows' pages, in every pass's cache layers alike."""
    from pyre_b200.engine import replay as rp
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.models.model import load_model
    standins.install(monkeypatch)
    d, _reqs, _plain = folders["A"]
    model, _ = load_model(d, "cpu", "float32")
    cache, stepper = rp.runtime_for_model(model, 256, 16, 4, cuda_graphs=False)
    ids = H.random_ids(300, 90, seed=3)
    cache.begin("w")
    stepper.step([StepEntry("w", ids[:70], [69])])
    for t in ids[70:]:
        stepper.step([StepEntry("w", [t], [0])])
    held = {g.spec.window: g.pages_held("w") for g in cache.groups}
    assert held == {11: 1, 23: 2}, held        # positions 79..89 and 67..89 on pages of 16
    cache.end("w")
    cache.check()


def test_a_layer_without_a_feed_forward_may_hold_its_second_gain(tmp_path, monkeypatch, folders):
    """The random mode leaves the unused gain out; a checkpoint that holds it loads as well and computes the same."""
    from safetensors.torch import load_file, save_file
    from pyre_b200.models.model import load_model
    standins.install(monkeypatch)
    d, _reqs, _plain = folders["A"]
    state = load_file(str(d / "model.safetensors"))
    assert "l2.ls2" not in state
    state["l2.ls2"] = torch.full((96,), 3.0)
    (tmp_path / "config.json").write_text((d / "config.json").read_text())
    save_file(state, str(tmp_path / "model.safetensors"))
    model, _ = load_model(tmp_path, "cpu", "float32")
    assert model.loaded and model.blocks[2].gain2 is None


def test_random_model_folder_loads(tmp_path, monkeypatch):
    from pyre_b200.models.model import load_model
    from pyre_b200.weights import write_random_model

    standins.install(monkeypatch)
    cfg = config_from_dict(PH.PIV_B)
    write_random_model(tmp_path, cfg, seed=1)
    assert json.loads((tmp_path / "config.json").read_text())["architecture"] == "Pivinex"
    model, loaded = load_model(tmp_path, "cpu", "float32")
    assert loaded == cfg and model.loaded
