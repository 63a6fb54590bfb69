"""``Vizalix`` described as an arrangement of parts.

A decoder whose layers each pair one of three mixers with a dense gated feed-forward (or none), both reading
the same normalised residual (``x <- x + mixer(norm1(x)) + ff(norm2(x))``, norms with a single gain):

* ``channel_delta``  gated delta rule with a decay per head and key channel (``channel_gated_delta``)
* ``attention``      windowed attention with partial, wavelength-scaled rotary positions, capped scores and
                     a mix of the heads' scores before the softmax (``head_mix_attention``)
* ``mamba2``         state-space recurrence (``mamba2``)

A stretch of the layers may run several times in a row with the same weights; every pass has caches and
states of its own (the schedule names a layer several times) and opens with a run that mixes the
embedding's output back into the residual (``stream_merge``), whose weights all passes share.

Nothing here computes: the function turns ``config.json`` into a :class:`ModelSpec`.  The ranks of the
low-rank decay and gate projections of ``channel_delta`` are given by the shapes of ``a1`` and ``g1`` alone:
a folder's checkpoint header is read for them (``tensor_shapes``), else ``decay_rank`` / ``gate_rank`` of the
mixer's sizes, else a default.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Optional, Tuple

from ..config.registry import register_architecture
from ..config.spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.vizalix_config import VizalixConfig

DEFAULT_LOW_RANK = 16


def _rank(mixer: Mapping[str, Any], key: str, name: str, shapes: Optional[Mapping[str, Tuple[int, ...]]]) -> int:
    if shapes is not None and name in shapes:
        return int(shapes[name][0])
    return int(mixer.get(key, DEFAULT_LOW_RANK))


def _mixer_spec(c: VizalixConfig, i: int, shapes) -> PartSpec:
    l = c.layers[i]
    m, W = l.mixer, c.width
    if l.type == "channel_delta":
        return PartSpec("channel_gated_delta", {
            "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "conv": m["conv"], "eps": c.eps,
            "decay_rank": _rank(m, "decay_rank", f"l{i}.mix.a1", shapes),
            "gate_rank": _rank(m, "gate_rank", f"l{i}.mix.g1", shapes)})
    if l.type == "attention":
        position = PartSpec("none")
        rot = m.get("rot")
        if rot:
            params = {"head_dim": m["dim"], "rot_dim": rot["dims"], "theta": rot["base"]}
            sc = rot.get("scaling")
            if sc:
                params.update({k: sc[k] for k in ("factor", "low", "high", "original")})
            position = PartSpec("rope_scaled" if sc else "rope", params)
        return PartSpec("head_mix_attention", {
            "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "window": m["mask"]["size"], "scale": m["scale"],
            "softcap": m.get("softcap", 0.0), "position": position,
            # every attention layer of the design mixes its heads' scores; a checkpoint header that was read
            # and lacks the matrix says otherwise
            "head_mix": shapes is None or f"l{i}.mix.talk" in shapes})
    return PartSpec("mamba2", {
        "hidden_size": W, "num_heads": m["heads"], "head_dim": m["vdim"], "state_size": m["state"],
        "groups": m.get("groups", 1), "norm_groups": m.get("norm_groups", 1), "conv": m["conv"], "eps": c.eps})


def build_vizalix(config_json: Dict[str, Any]) -> ModelSpec:
    c = VizalixConfig.from_json_dict(config_json)
    shapes = config_json.get("tensor_shapes")
    W = c.width
    layers = []
    for i, l in enumerate(c.layers):
        parts = {
            "mixer_norm": LayerPart("norm", PartSpec("rmsnorm_scalar", {"eps": c.eps, "tensor": "norm1"}), ""),
            "mixer": LayerPart("mixer", _mixer_spec(c, i, shapes), "mix."),
        }
        if l.ff is not None:
            parts["feed_forward_norm"] = LayerPart("norm", PartSpec("rmsnorm_scalar", {"eps": c.eps, "tensor": "norm2"}), "")
            parts["feed_forward"] = LayerPart("feed_forward", PartSpec("gated_mlp", {
                "hidden_size": W, "intermediate_size": l.ff, "activation": "gelu_tanh",
                "gate": "gate", "up": "up", "down": "down"}), "mlp.")
        layers.append(LayerSpec(f"l{i}", PartSpec("parallel_residual", {"feed_forward": l.ff is not None}), parts))
    schedule = []
    merge = None
    if c.loop is not None:
        merge = len(layers)
        layers.append(LayerSpec("loop", PartSpec("stream_merge", {"hidden_size": W, "passes": c.loop.times,
                                                                  "weight": "in", "step": "step"}), {}))
    for i, opens_pass in c.runs():
        if opens_pass is not None:
            schedule.append(ScheduleEntry(merge, args={"pass": opens_pass, "auxiliary": True}))
        schedule.append(ScheduleEntry(i))
    return ModelSpec(
        architecture=c.architecture, hidden_size=W, vocab_size=c.vocab, max_context=1 << 30,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": W, "tensor": "embed"}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm_scalar", {"eps": c.eps, "tensor": "final.norm"}),
        lm_head=PartSpec("linear", {"vocab_size": c.vocab, "hidden_size": W, "tied_to": None, "tensor": "head"}),
        embedding_prefix="", final_norm_prefix="", lm_head_prefix="")


register_architecture("Vizalix", build_vizalix,
                      "Vizalix decoder (parallel residual layers with scalar RMS norms; channel-wise gated delta "
                      "rule, windowed head-mixing attention or Mamba-2 mixers; gelu-gated feed-forward; a looped "
                      "stretch of layers that re-reads the embedding)")
