"""Silupel on a machine without a GPU: configuration and plan, what is computed on the host (the stretched rotation table,
the order of layer runs, the reordering of latent attention's rotated rows), and the engine's host side (batching, the token
shift's row and the recurrence's state carried from step to step, a cache and a state per layer run) with the torch
stand-in for the CUDA library against the plain implementation."""
import copy

import numpy as np
import pytest
import torch

import plain_silupel as plain
import traces
from silupel_util import BLOCKS, CONFIGS, att, gru, lat, layer, make_folder, model, plain_logits, requests


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(c, str(tmp_path_factory.mktemp(f"silupel_{n}")), 11 + i) for i, (n, c) in enumerate(CONFIGS.items())}


def test_plan_follows_the_layer_list_and_the_loop():
    from hfcpu_b200.config import config_from_dict, SilupelConfig
    cfg = config_from_dict(CONFIGS["odd"])
    assert isinstance(cfg, SilupelConfig)
    plan = cfg.plan()
    assert [l.mixer.kind for l in plan.layers] == ["mingru", "paged_attention", "latent_attention", "mingru", "paged_attention",
                                                   "latent_attention"]
    assert [e.layer for e in plan.schedule] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4, 5] == plain.run_order(CONFIGS["odd"])
    assert all(e.cache_of is None for e in plan.schedule)                    # every run keeps its own cache
    assert [l.mixer.args.get("chunk") for l in plan.layers] == [None, 12, None, None, 50, None]
    assert [l.mixer.args.get("softcap") for l in plan.layers] == [None, 7.0, None, None, 30.0, None]
    assert [l.ffn.kind if l.ffn else None for l in plan.layers] == ["gated", "gated", None, "gated", None, "gated"]
    assert all(l.ffn.args["activation"] == "gelu_tanh" for l in plan.layers if l.ffn)
    assert all(l.norm1.kind == "layernorm" for l in plan.layers) and plan.final_norm.kind == "layernorm"
    assert all(l.block.kind == "prenorm_residual" and l.block.args["token_shift"] == f"l{i}.shift" for i, l in enumerate(plan.layers))
    assert plan.layers[1].mixer.args["head_scale_tensor"] == "temp" and plan.layers[1].mixer.args["out_gate"]["kind"] == "sigmoid"
    assert len(plan.positions) == 4 and all(p.args["pairing"] == "half" for p in plan.positions.values())
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    assert [e.layer for e in config_from_dict(CONFIGS["wide"]).plan().schedule] == [0, 1, 0, 1, 2, 3, 4, 5]
    assert [e.layer for e in config_from_dict(CONFIGS["thin"]).plan().schedule] == [0, 1, 2, 3, 4]
    once = copy.deepcopy(CONFIGS["odd"])
    once["loop"] = {"start": 2, "stop": 2, "times": 5}                        # an empty stretch
    assert [e.layer for e in config_from_dict(once).plan().schedule] == list(range(6))


def test_configuration_errors():
    from hfcpu_b200.config import ConfigError, UnsupportedError, config_from_dict
    bad = copy.deepcopy(CONFIGS["thin"])
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(UnsupportedError, match="convolution"):
        config_from_dict(bad)
    bad = copy.deepcopy(CONFIGS["thin"])
    bad["loop"] = {"start": 3, "stop": 9, "times": 2}
    with pytest.raises(ConfigError, match="loop"):
        config_from_dict(bad)
    bad = copy.deepcopy(CONFIGS["thin"])
    bad["layers"][2]["mixer"]["rot"]["dims"] = 2
    with pytest.raises(UnsupportedError, match="rot_dim"):
        config_from_dict(bad)
    bad = copy.deepcopy(CONFIGS["thin"])
    del bad["layers"][1]["mixer"]["width"]
    with pytest.raises(ConfigError, match="width"):
        config_from_dict(bad)


def test_tensor_names():
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    specs = {s.name: s for s in build_model_specs(config_from_dict(CONFIGS["odd"]))}
    assert specs["embed"].shape == (211, 72) and specs["head"].shape == (211, 72) and specs["final.norm"].shape == (72,)
    assert all(specs[f"l{i}.shift"].shape == (72,) and specs[f"l{i}.norm1"].shape == (72,) for i in range(6))
    assert specs["l0.mix.z"].shape == (100, 72) and specs["l0.mix.x.b"].shape == (100,) and specs["l0.mix.o"].shape == (72, 100)
    assert specs["l0.mix.g"].shape == (100, 72) and "l0.mix.g.b" not in specs
    assert specs["l1.mix.q"].shape == (144, 72) and specs["l1.mix.k.b"].shape == (72,) and specs["l1.mix.v"].shape == (120, 72)
    assert specs["l1.mix.g"].shape == (240, 72) and specs["l1.mix.o"].shape == (72, 240) and specs["l1.mix.o.b"].shape == (72,)
    assert specs["l1.mix.temp"].shape == (6,)
    assert specs["l2.mix.dq"].shape == (40, 72) and specs["l2.mix.uq"].shape == (72, 40) and specs["l2.mix.dkv"].shape == (32, 72)
    assert specs["l2.mix.dkv.norm"].shape == (24,) and specs["l2.mix.uk"].shape == (48, 24) and specs["l2.mix.uv"].shape == (72, 24)
    assert specs["l2.norm2"].optional and "l2.mlp.up" not in specs and not specs["l1.norm2"].optional
    assert specs["l1.mlp.gate"].shape == (64, 72) and specs["l1.mlp.down"].shape == (72, 64)


@pytest.mark.parametrize("rot", [{"dims": 32, "base": 50000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}},
                                 {"dims": 8, "base": 500.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}},
                                 {"dims": 12, "base": 77.0, "scaling": {"factor": 2.0, "low": 0.5, "high": 2.0, "original": 16}},
                                 {"dims": 16, "base": 10000.0}])
def test_rotation_table_stretched_by_wavelength(rot):
    """All three ranges occur: frequencies kept, divided, and blended between."""
    from hfcpu_b200.parts.rotary import Rotary
    r = Rotary(rot["dims"], rot["dims"], rot["base"], "half", rot.get("scaling"))
    f, magnitude = r.frequencies()
    want = plain.rot_frequencies(rot)
    assert magnitude == 1.0 and np.allclose(f.numpy(), want, rtol=1e-14, atol=0)
    if "scaling" in rot:
        base = plain.rot_frequencies({"dims": rot["dims"], "base": rot["base"]})
        ratio = want / base
        assert ratio.max() == 1.0 and np.isclose(ratio.min(), 1.0 / rot["scaling"]["factor"])
        assert ((ratio < 1.0) & (ratio > 1.0 / rot["scaling"]["factor"] * 1.0001)).any()
    r.prepare(50, torch.device("cpu"))
    ang = np.arange(50)[:, None] * want[None, :]
    assert np.allclose(r.cos_sin.numpy(), np.stack([np.cos(ang), np.sin(ang)], -1), atol=1e-6)


def test_latent_rows_are_reordered_for_the_kernels_pairing():
    """The rotated rows of the two projections go from (i, i + half) to (2i, 2i + 1); everything else stays."""
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.parts import make_part
    rot = make_part("position", PartSpec("rotary", {"head_dim": 6, "n_rot": 6, "theta": 10.0, "pairing": "half"}))
    part = make_part("mixer", PartSpec("latent_attention", {
        "hidden_size": 5, "num_heads": 2, "head_dim": 3, "rot_dim": 6, "v_head_dim": 4, "q_rank": 7, "kv_rank": 2, "scale": 1.0,
        "norm_eps": 1e-6, "window": 0, "position": "r", "prefix": "m"}), positions={"r": rot})
    g = torch.Generator().manual_seed(0)
    tensors = {s.name: torch.randn(s.shape, generator=g) for s in part.tensor_specs()}
    part.bind(tensors, torch.float32, torch.device("cpu"))
    order = [0, 3, 1, 4, 2, 5]
    assert torch.equal(part.w_down[:9], torch.cat([tensors["m.dq"], tensors["m.dkv"][:2]]))
    assert torch.equal(part.w_down[9:], tensors["m.dkv"][2:][order])
    uq = tensors["m.uq"].view(2, 9, 7)
    assert torch.equal(part.w_uq.view(2, 9, 7)[:, :3], uq[:, :3]) and torch.equal(part.w_uq.view(2, 9, 7)[:, 3:], uq[:, 3:][:, order])


LENGTHS = {"odd": [1, 19, 40, 27], "wide": [3, 70, 20], "thin": [2, 9, 41]}


@pytest.mark.parametrize("family", ["whole", "portions", "mixed"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_engine_host_side_matches_plain(folders, name, family):
    """Every cutting through the engine (pages, slots, the shift's previous row, the recurrence's state, a cache per run of
    a looped layer) with the stand-in kernels gives the plain implementation's logits."""
    import hfcpu_b200
    from emu_backend import EmuBackend
    from hfcpu_b200 import kernels
    old = kernels._backend
    kernels.set_backend(EmuBackend())
    try:
        reqs = requests(CONFIGS[name]["vocab"], LENGTHS[name], seed=4)
        steps = {"whole": traces.whole, "portions": lambda r: traces.portions(r, sizes=(7, 2, 16, 3, 5, 2, 11)),
                 "mixed": lambda r: traces.mixed(r, max_live=3, prefill_sizes=(9, 2, 5, 17))}[family](reqs)
        m = hfcpu_b200.load_model(folders[name], torch.float32, "cpu")
        eng = hfcpu_b200.Engine(m, block_size=BLOCKS[name], max_tokens=traces.peak_tokens(steps, round_to=BLOCKS[name]), max_requests=3)
        assert len(eng.slots.tensors) >= len(m.plan.schedule)                 # a shift row per run, and the recurrences' states
        got = traces.run_in_process(eng, steps, check=eng.cache.check)
        assert eng.cache.pages_in_use() == 0 and eng.slots.free_count == 3
        for (r, pos), row in got.items():
            want = plain_logits(folders[name], reqs[r])[pos]
            assert float((row.double() - want).abs().max() / want.abs().max()) < 2e-4, (r, pos)
    finally:
        kernels.set_backend(old)


def test_a_slot_taken_over_starts_from_zero(folders):
    """A request that gets the slot of a finished one must not see its shift row or recurrent state."""
    import hfcpu_b200
    from emu_backend import EmuBackend
    from hfcpu_b200 import kernels
    old = kernels._backend
    kernels.set_backend(EmuBackend())
    try:
        m = hfcpu_b200.load_model(folders["thin"], torch.float32, "cpu")
        eng = hfcpu_b200.Engine(m, block_size=4, max_tokens=64, max_requests=1)
        ids = requests(97, [11, 11], seed=9)
        for r in ("r0", "r1"):
            eng.add_request(r)
            a = eng.step([hfcpu_b200.StepEntry(r, ids[r][:6], [5])])[0].clone()
            b = eng.step([hfcpu_b200.StepEntry(r, ids[r][6:], [4])])[0].clone()
            eng.finish_request(r)
            want = plain_logits(folders["thin"], ids[r])
            assert float((a.double() - want[5]).abs().max()) < 1e-3 and float((b.double() - want[10]).abs().max()) < 1e-3
    finally:
        kernels.set_backend(old)
