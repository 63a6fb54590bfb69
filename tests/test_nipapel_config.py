"""Nipapel on the CPU: the configuration reader, the model description built from it, the manifest of tensors,
how layers share caches and how long a cache keeps a token, and the plain model's own consistency."""

import copy

import pytest
import torch

import nipapel_tiny as nt
import plain_nipapel as pn


def test_the_description_follows_the_configuration():
    from mini_infer_b200.config import build_model_spec
    from mini_infer_b200.engine.model import Model
    for name, cfg in nt.CONFIGS.items():
        spec = build_model_spec(cfg)
        assert [e.layer for e in spec.schedule] == list(range(len(cfg["layers"])))
        assert [e.cache_from for e in spec.schedule] == [l["mixer"].get("kv_from") for l in cfg["layers"]]
        model = Model(spec)
        # every layer that does not borrow has a cache of its own
        owners = sum(g.num_layers for g in model.kv_groups)
        assert owners == sum(1 for l in cfg["layers"] if l["mixer"].get("kv_from") is None)
        assert not model.state_needs
        # the engine's manifest is exactly what the configuration implies
        want = nt.make_weights(cfg, 0)
        decl = {d.name: tuple(d.shape) for d in model.tensor_decls()}
        assert decl == {k: tuple(v.shape) for k, v in want.items()}, name


def test_a_borrowed_cache_keeps_tokens_for_its_widest_reader():
    from mini_infer_b200.config import build_model_spec
    from mini_infer_b200.engine.model import Model
    model = Model(build_model_spec(nt.CONFIG_A))
    latent = [g for g in model.kv_groups if hasattr(g.need, "rank")]
    assert [(g.need.rank, g.need.rot_dim, g.need.window, g.num_layers) for g in latent] == [(20, 4, 13, 1)]
    assert model.bindings[2]["mixer"].writes is False and model.bindings[1]["mixer"].writes is True
    assert (model.bindings[2]["mixer"].group, model.bindings[2]["mixer"].layer_slot) == \
        (model.bindings[1]["mixer"].group, model.bindings[1]["mixer"].layer_slot)
    # a narrower reader leaves its owner's window as it is
    model = Model(build_model_spec(nt.CONFIG_B))
    assert sorted(g.need.window for g in model.kv_groups if hasattr(g.need, "rank")) == [1, 64]
    kv = sorted((g.need.window, g.need.keep_first, g.need.head_dim, g.need.value_dim) for g in model.kv_groups
                if hasattr(g.need, "head_dim"))
    assert kv == [(1, 1, 20, 96), (5, 9, 24, 40)]


def test_pages_of_kept_first_tokens_are_never_given_back():
    from mini_infer_b200.cache import CacheGroupSpec, CacheManager, KVNeed
    groups = [CacheGroupSpec(KVNeed(1, 8, window=6, keep_first=5), ("a",)), CacheGroupSpec(KVNeed(1, 8, window=6), ("b",))]
    cm = CacheManager(groups, [32, 32], page_size=4, num_slots=2)
    cm.add_request("x")
    for n in (7, 2, 30, 1, 1, 1, 9):
        cm.reserve("x", n)
        cm.commit("x")
        cm.check_invariants()
    kept, plain = cm.block_table(0, "x"), cm.block_table(1, "x")
    total = cm.num_tokens("x")
    first_needed = (total - 6 + 1) // 4
    assert kept[0] >= 0 and kept[1] >= 0                     # tokens 0..4 live in pages 0 and 1
    assert all(p < 0 for p in kept[2:first_needed]) and all(p >= 0 for p in kept[first_needed:])
    assert all(p < 0 for p in plain[:first_needed]) and all(p >= 0 for p in plain[first_needed:])
    cm.release("x")
    assert cm.used_pages() == [0, 0]


@pytest.mark.parametrize("damage", [
    lambda c: c.pop("width"), lambda c: c["layers"][0].update(type="conv"),
    lambda c: c["layers"][0]["mixer"].pop("mask"), lambda c: c["layers"][0]["mixer"].pop("scale"),
    lambda c: c["layers"][0]["mixer"].update(kv_heads=3), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][1]["mixer"]["mask"].update(keep_first=2),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=2),
    lambda c: c["layers"][2]["mixer"].update(kv_from=3), lambda c: c["layers"][2]["mixer"].update(kv_from=0),
    lambda c: c["layers"][2]["mixer"].update(kv_rank=8),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=6), lambda c: c["layers"][0]["mlp"].pop("limit"),
    lambda c: c["layers"][3].update(mlp={"kind": "sparse", "ff": 8}), lambda c: c["norm"].pop("eps")])
def test_a_damaged_configuration_is_refused(damage):
    from mini_infer_b200.config import ConfigError, build_model_spec
    cfg = copy.deepcopy(nt.CONFIG_A)
    damage(cfg)
    with pytest.raises(ConfigError):
        build_model_spec(cfg)


def test_plain_model_prefix_property():
    """Causal: the logits of a prefix do not change when tokens follow."""
    for name, cfg in nt.CONFIGS.items():
        w = nt.make_weights(cfg, 3)
        toks = nt.random_requests(cfg, [40], 5)["r0"]
        full = pn.forward(cfg, w, toks)
        part = pn.forward(cfg, w, toks[:23])
        assert torch.allclose(full[:23], part, atol=1e-9), name


def test_plain_window_and_kept_first_edges_matter():
    """A key that stands out moves the plain attention's output when it is the last one inside the window or
    the last of the kept first keys, and not at all just outside either."""
    T, d, e, W, F = 30, 8, 4, 7, 3
    g = torch.Generator().manual_seed(0)
    q = torch.zeros(T, 1, d, dtype=torch.float64)
    k = torch.randn(T, 1, d, generator=g, dtype=torch.float64) * 0.01
    v = torch.randn(T, 1, e, generator=g, dtype=torch.float64)
    q[-1, 0, 0] = 30.0
    for key, seen in ((T - 1 - (W - 1), True), (T - 1 - W, False), (F - 1, True), (F, False)):
        kk = k.clone()
        kk[key, 0, 0] = 1.0
        o = pn.masked_softmax_attention(q, kk, v, 1.0, pn.visible(T, W, F))[-1, 0]
        assert bool(torch.allclose(o, v[key, 0], atol=1e-6)) == seen, key


def test_plain_latent_attention_equals_attention_over_the_unfolded_keys_and_values():
    """The plain latent mixer forms every head's keys and values; folding the key matrices into the queries and
    applying the value matrices after the weighted sum gives the same output."""
    cfg = nt.CONFIG_A
    w = {k: v.double() for k, v in nt.make_weights(cfg, 4).items()}
    m, p = cfg["layers"][1]["mixer"], "l1.mix."
    T = 19
    h = torch.randn(T, cfg["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    kept = pn.latent_of(h, w, p, m, 1e-5)
    want = pn.latent_attention_mixer(h, w, p, m, 1e-5, kept)
    H, d, r, e, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    lat, kr = kept
    q = (pn.norm_plain(h @ w[p + "dq"].T, w[p + "dq.norm"], 1e-5) @ w[p + "uq"].T).view(T, H, d + r)
    folded = torch.einsum("thd,hdc->thc", q[..., :d], w[p + "uk"].view(H, d, c))
    qq = torch.cat([folded, pn.rotate_neighbours(q[..., d:], r, m["rot"]["base"])], dim=-1)
    rows = torch.cat([lat, kr], dim=-1)[:, None, :]
    o = pn.masked_softmax_attention(qq, rows, lat[:, None, :], m["scale"], pn.visible(T, m["mask"]["size"]))
    v = torch.einsum("thc,hec->the", o, w[p + "uv"].view(H, e, c)).reshape(T, H * e)
    got = (v * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T
    assert torch.allclose(got, want, atol=1e-9)


def test_plain_router_weights_are_the_softmax_over_the_chosen_logits():
    cfg = nt.CONFIG_A
    w = {k: v.double() for k, v in nt.make_weights(cfg, 2).items()}
    h = torch.randn(6, cfg["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    rec = []
    pn.routed_ff(h, w, "l1.mlp.", cfg["layers"][1]["mlp"], chosen=rec)
    idx, z = rec[0]
    assert idx.shape == (6, 2)
    assert torch.equal(torch.sort(idx, dim=1).values, torch.sort(torch.topk(z, 2, dim=1).indices, dim=1).values)
    # the bias takes part in the choice: a large bias on one expert makes every token choose it
    w["l1.mlp.router.b"] = torch.tensor([0.0, 0.0, 50.0, 0.0, 0.0], dtype=torch.float64)
    rec = []
    pn.routed_ff(h, w, "l1.mlp.", cfg["layers"][1]["mlp"], chosen=rec)
    assert bool((rec[0][0] == 2).any(dim=1).all())


def test_a_model_names_the_kernel_sources_it_needs():
    """What a first call in a fresh checkout compiles: the sources of the model's parts and the engine's own."""
    from mini_infer_b200.config import build_model_spec
    from mini_infer_b200.csrc import build as B
    from mini_infer_b200.engine.model import Model
    from mini_infer_b200.ops.library import ENGINE_SOURCES
    files = set(Model(build_model_spec(nt.CONFIG_A)).kernel_files())
    assert {"attention_latent.cu", "attention_mix.cu", "attention_prefill_tc.cu", "moe.cu", "residual_forms.cu"} <= files
    assert not files & {"recurrent.cu", "attention.cu", "attention_prefill.cu"}
    assert files | set(ENGINE_SOURCES) <= set(B.sources())
    # a partial build always holds the core; all sources together are the whole library; unknown names are refused
    assert B._subset(["moe.cu"]) == sorted({"moe.cu", *B.CORE})
    assert B._subset(B.sources()) is None and B._subset(None) is None
    with pytest.raises(ValueError):
        B._subset(["no_such_kernels.cu"])
    assert B._paths("/x", None)[0] != B._paths("/x", ["elementwise.cu", "moe.cu"])[0]
