"""Vizalix on the CPU: the configuration reader, the model description built from it, the manifest of
tensors, the rescaled rotary frequencies, and the plain model's own consistency."""

import copy
import math

import pytest
import torch

import plain_vizalix as pv
import vizalix_tiny as vt


def test_the_description_follows_the_configuration():
    from mini_infer_b200.config import build_model_spec
    from mini_infer_b200.engine.model import Model
    for name, cfg in vt.CONFIGS.items():
        spec = build_model_spec(cfg)
        runs = pv.layer_runs(cfg)
        merges = [e for e in spec.schedule if e.args.get("auxiliary")]
        layers = [e.layer for e in spec.schedule if not e.args.get("auxiliary")]
        assert layers == [i for i, _ in runs]
        assert [e.args["pass"] for e in merges] == [t for _, t in runs if t is not None]
        model = Model(spec)
        # every run of a layer has a cache or a state of its own
        kv = sum(g.num_layers for g in model.kv_groups)
        assert kv + len(model.state_needs) == len(runs)
        # the engine's manifest is exactly what the configuration implies
        want = vt.make_weights(cfg, 0)
        decl = {d.name: tuple(d.shape) for d in model.tensor_decls()}
        assert decl == {k: tuple(v.shape) for k, v in want.items()}, name


def test_layers_with_other_windows_or_sizes_get_cache_groups_of_their_own():
    from mini_infer_b200.config import build_model_spec
    from mini_infer_b200.engine.model import Model
    model = Model(build_model_spec(vt.CONFIG_P))
    assert sorted((g.need.window, g.need.head_dim, g.need.value_dim, g.num_layers) for g in model.kv_groups) == \
        [(9, 16, 8, 1), (33, 12, 20, 1)]
    assert len(model.state_needs) == 6      # two layers in three passes


def test_low_ranks_come_from_the_checkpoint_header_first():
    from mini_infer_b200.config import build_model_spec
    cfg = copy.deepcopy(vt.CONFIG_Q)
    del cfg["layers"][0]["mixer"]["decay_rank"]
    cfg["tensor_shapes"] = {"l0.mix.a1": (11, 72), "l0.mix.g1": (2, 72)}
    m = build_model_spec(cfg).layers[0].mixer
    assert (m.get("decay_rank"), m.get("gate_rank")) == (11, 2)


@pytest.mark.parametrize("damage", [
    lambda c: c.pop("width"), lambda c: c["layers"][0].update(type="conv"),
    lambda c: c["layers"][0]["mixer"].pop("mask"), lambda c: c.update(loop={"start": 2, "stop": 1, "times": 1}),
    lambda c: c["layers"][1]["mixer"].update(kv_heads=3), lambda c: c["layers"][2].update(mlp={"kind": "sparse", "ff": 8}),
    lambda c: c["norm"].pop("eps"), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7)])
def test_a_damaged_configuration_is_refused(damage):
    from mini_infer_b200.config import ConfigError, build_model_spec
    cfg = copy.deepcopy(vt.CONFIG_P)
    damage(cfg)
    with pytest.raises(ConfigError):
        build_model_spec(cfg)


def test_rescaled_frequencies():
    from mini_infer_b200.config import PartSpec, part_class
    rot = {"base": 300.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 40}}
    cls = part_class("position", "rope_scaled")
    part = cls({"head_dim": 24, "rot_dim": 16, "theta": 300.0, **rot["scaling"]}, "")
    got = part.table("cpu").double()
    want = pv.rotary_frequencies(rot)
    assert torch.allclose(got, want, rtol=1e-6)
    plain = torch.tensor([300.0 ** (-2 * i / 16) for i in range(8)], dtype=torch.float64)
    # the three regimes are all met: kept, divided, blended
    ratio = (want / plain).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 8) < 1e-12 and any(1 / 8 + 1e-6 < r < 1 - 1e-6 for r in ratio)


def test_plain_model_prefix_property():
    """Causal: the logits of a prefix do not change when tokens follow (every mechanism looks back only)."""
    for name, cfg in vt.CONFIGS.items():
        w = vt.make_weights(cfg, 3)
        toks = vt.random_requests(cfg, [40], 5)["r0"]
        full = pv.forward(cfg, w, toks)
        part = pv.forward(cfg, w, toks[:23])
        assert torch.allclose(full[:23], part, atol=1e-9), name


def test_plain_window_edge_matters():
    """A key that stands out moves the plain attention's output when it is the last one inside the window
    and not at all when it is the first one outside."""
    T, d, e, W = 30, 8, 4, 7
    g = torch.Generator().manual_seed(0)
    q = torch.zeros(T, 1, d, dtype=torch.float64)
    k = torch.randn(T, 1, d, generator=g, dtype=torch.float64) * 0.01
    v = torch.randn(T, 1, e, generator=g, dtype=torch.float64)
    q[-1, 0, 0] = 30.0
    for dist, seen in ((W - 1, True), (W, False)):
        kk = k.clone()
        kk[T - 1 - dist, 0, 0] = 1.0
        o = pv.mixed_head_attention(q, kk, v, 1.0, None, None, W)[-1, 0]
        assert bool(torch.allclose(o, v[T - 1 - dist, 0], atol=1e-6)) == seen
