"""``Nipapel`` described as an arrangement of parts.

A decoder whose layers read ONE normalised residual with both of their parts
(``x <- x + mixer(h) + ff(h)``, ``h = norm(x)``; norms whose stored weight is the gain's offset from one; the
embedding's rows go through such a norm as well before they become the residual):

* ``attention``          grouped-query attention whose query and key heads are brought to unit root mean
                         square (with a gain per dimension), rotated in part, behind a window that keeps
                         the first tokens of a request visible (``head_mix_attention`` without a head mix)
* ``latent_attention``   attention through a latent per token with a gate on the heads' outputs; a layer may
                         read the latents an earlier layer caches (``latent_attention``; the schedule
                         entry's ``cache_from``)

and a feed-forward whose gated units bound both halves (``clamped_swish``): dense (``gated_mlp``), a
mixture of experts with a router bias and weights that are the softmax over the chosen logits
(``sparse_moe``), or none.  Nothing here computes: the function turns ``config.json`` into a
:class:`ModelSpec`.
"""

from __future__ import annotations

from typing import Any, Dict

from ..config.nipapel_config import NipapelConfig
from ..config.registry import register_architecture
from ..config.spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _norm(c: NipapelConfig, tensor: str) -> PartSpec:
    return PartSpec("rmsnorm", {"size": c.width, "eps": c.eps, "tensor": tensor, "one_plus": True})


def _mixer_spec(c: NipapelConfig, i: int) -> PartSpec:
    l = c.layers[i]
    m, W = l.mixer, c.width
    if l.type == "attention":
        position = PartSpec("none")
        rot = m.get("rot")
        if rot:
            position = PartSpec("rope", {"head_dim": m["dim"], "rot_dim": rot["dims"], "theta": rot["base"]})
        return PartSpec("head_mix_attention", {
            "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "window": m["mask"]["size"], "keep_first": m["mask"].get("keep_first", 0),
            "scale": m["scale"], "head_mix": False, "qk_norm": {"eps": c.eps}, "position": position})
    rot = m["rot"]
    return PartSpec("latent_attention", {
        "hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
        "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "window": m["mask"]["size"],
        "scale": m["scale"], "eps": c.eps, "shares_cache": m.get("kv_from") is not None,
        "position": PartSpec("rope", {"head_dim": m["rot_dim"], "rot_dim": rot["dims"], "theta": rot["base"]})})


def _ff_spec(c: NipapelConfig, i: int) -> PartSpec:
    mlp = c.layers[i].mlp
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"hidden_size": c.width, "intermediate_size": mlp["ff"],
                                      "activation": "clamped_swish", "limit": mlp["limit"],
                                      "gate": "gate", "up": "up", "down": "down"})
    return PartSpec("sparse_moe", {
        "hidden_size": c.width, "num_experts": mlp["router"]["experts"], "top_k": mlp["router"]["top"],
        "expert_intermediate_size": mlp["expert"]["ff"], "norm_topk_prob": True,
        "activation": "clamped_swish", "limit": mlp["expert"]["limit"],
        "router": "router", "router_bias": True, "router_bias_name": "router.b", "expert": "e{e}.",
        "gate": "gate", "up": "up", "down": "down"})


def build_nipapel(config_json: Dict[str, Any]) -> ModelSpec:
    c = NipapelConfig.from_json_dict(config_json)
    W = c.width
    layers, schedule = [], []
    for i, l in enumerate(c.layers):
        parts = {"mixer_norm": LayerPart("norm", _norm(c, "norm1"), ""),
                 "mixer": LayerPart("mixer", _mixer_spec(c, i), "mix.")}
        if l.mlp is not None:
            parts["feed_forward"] = LayerPart("feed_forward", _ff_spec(c, i), "mlp.")
        layers.append(LayerSpec(f"l{i}", PartSpec("parallel_residual", {"feed_forward": l.mlp is not None,
                                                                        "shared_norm": True}), parts))
        # layers run once each, in order: a schedule position is a layer's index
        schedule.append(ScheduleEntry(i, cache_from=l.mixer.get("kv_from")))
    return ModelSpec(
        architecture=c.architecture, hidden_size=W, vocab_size=c.vocab, max_context=1 << 30,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": W, "tensor": "embed",
                                               "norm": _norm(c, "embed.norm")}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=_norm(c, "final.norm"),
        lm_head=PartSpec("linear", {"vocab_size": c.vocab, "hidden_size": W, "tied_to": None, "tensor": "head"}),
        embedding_prefix="", final_norm_prefix="", lm_head_prefix="")


register_architecture("Nipapel", build_nipapel,
                      "Nipapel decoder (layers whose mixer and feed-forward read one offset-gain RMS norm; "
                      "windowed grouped-query attention with normalised heads and kept first tokens, or attention "
                      "through shared latents with an output gate; dense or routed feed-forward with bounded "
                      "gated units)")
