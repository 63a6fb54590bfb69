"""Tiny Vizalix configurations and weights for the tests.

The configurations differ from one another in every size and option: order and kinds of layers, layers
without a feed-forward, a looped stretch in the middle, over all layers or none, one pass or three, key and
value sizes that differ, one head, as many key heads as heads or fewer, windows of 1, 9 and more than a
prompt, rotation of part of a head or all of it, with and without rescaled frequencies and score cap,
convolutions of 2, 3 and 4 taps, one or several B/C groups and norm groups.  Weights are drawn so that
activations stay of order one (a model whose mixers put out almost nothing hides their faults) and are
rounded to bfloat16, so that both precision paths and the plain model read the same numbers.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List

import torch


def _attn(heads, kv, dim, vdim, window, rot=None, cap=None, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window},
         "scale": scale if scale is not None else dim ** -0.5}
    if rot:
        m["rot"] = rot
    if cap:
        m["softcap"] = cap
    return m


CONFIG_P = {
    "architecture": "Vizalix", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 80},
         "mixer": _attn(4, 2, 16, 8, 9, rot={"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}, cap=5.0, scale=0.3)},
        {"type": "channel_delta", "mlp": None,
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 16, "conv": 3, "decay_rank": 5, "gate_rank": 6}},
        {"type": "mamba2", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"heads": 4, "vdim": 8, "state": 12, "groups": 2, "norm_groups": 2, "conv": 4}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 56},
         "mixer": _attn(2, 2, 12, 20, 33, rot={"base": 500.0, "dims": 12})},
    ],
    "loop": {"start": 1, "stop": 3, "times": 3},
}

CONFIG_Q = {
    "architecture": "Vizalix", "vocab": 131, "width": 72, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 24, "conv": 2, "decay_rank": 7, "gate_rank": 4}},
        {"type": "mamba2", "mlp": None,
         "mixer": {"heads": 6, "vdim": 10, "state": 9, "groups": 1, "norm_groups": 1, "conv": 2}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 100},
         "mixer": _attn(6, 3, 24, 40, 64, rot={"base": 250.0, "dims": 24, "scaling": {"factor": 2.0, "low": 1.0, "high": 8.0, "original": 32}}, cap=12.0)},
    ],
}

CONFIG_R = {
    "architecture": "Vizalix", "vocab": 64, "width": 40, "norm": {"eps": 3e-6},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 48}, "mixer": _attn(1, 1, 20, 96, 1, cap=2.0)},
        {"type": "mamba2", "mlp": {"kind": "dense", "ff": 48},
         "mixer": {"heads": 1, "vdim": 36, "state": 70, "groups": 1, "norm_groups": 3, "conv": 3}},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 72},
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 68, "vdim": 36, "conv": 4, "decay_rank": 3, "gate_rank": 3}},
        {"type": "attention", "mlp": None,
         "mixer": _attn(5, 1, 8, 8, 17, rot={"base": 1000.0, "dims": 4})},
    ],
    "loop": {"start": 0, "stop": 4, "times": 2},
}

# attention shapes that the bfloat16 path takes to the tensor cores (value size 64, key size a multiple of 16),
# once with more heads than one block finishes
CONFIG_T = {
    "architecture": "Vizalix", "vocab": 160, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mamba2", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"heads": 2, "vdim": 16, "state": 16, "groups": 2, "norm_groups": 1, "conv": 4}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 96},
         "mixer": _attn(4, 2, 32, 64, 40, rot={"base": 10000.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 2.0, "original": 48}}, cap=20.0)},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 32, "conv": 4, "decay_rank": 8, "gate_rank": 8}},
        {"type": "attention", "mlp": None, "mixer": _attn(36, 4, 16, 64, 23, cap=8.0)},
    ],
    "loop": {"start": 1, "stop": 4, "times": 2},
}

# one pass of a "loop" (the merge of the embedding still runs once)
CONFIG_S = dict(CONFIG_Q, loop={"start": 2, "stop": 3, "times": 1})

CONFIGS = {"P": CONFIG_P, "Q": CONFIG_Q, "R": CONFIG_R, "S": CONFIG_S, "T": CONFIG_T}


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """``name -> bfloat16 tensor`` for every tensor the configuration implies (names built here from the
    configuration alone, so the engine's own manifest is checked against an independent one)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def rnd(*shape, std=1.0):
        return torch.randn(*shape, generator=g) * std

    def lin(out, inn, gain=1.0):
        return rnd(out, inn, std=gain / math.sqrt(inn))

    w: Dict[str, torch.Tensor] = {"embed": rnd(cfg["vocab"], W), "head": lin(cfg["vocab"], W, 2.0),
                                  "final.norm": torch.tensor(1.0 + 0.2 * float(rnd(1)))}
    loop = cfg.get("loop")
    if loop:
        w["loop.in"] = lin(W, 2 * W, 1.4)
        w["loop.step"] = rnd(loop["times"], W, std=0.3)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = torch.tensor(1.0 + 0.2 * float(rnd(1)))
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            w[p + "norm2"] = torch.tensor(1.0 + 0.2 * float(rnd(1)))
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = lin(ff, W, 1.5), lin(ff, W, 1.5), lin(W, ff)
        q = p + "mix."
        if L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * d, W, 2.5), lin(G * d, W, 2.5), lin(G * e, W, 1.5)
            w[q + "talk"] = torch.eye(H) + rnd(H, H, std=0.3)
            w[q + "o"] = lin(W, H * e, 1.5)
        elif L["type"] == "channel_delta":
            H, G, d, e, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = m["decay_rank"], m["gate_rank"]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * e)):
                w[q + n] = lin(rows, W, 2.0)
                w[q + n + ".conv"] = rnd(rows, K, std=0.6)
            w[q + "b"] = lin(H, W, 2.0)
            w[q + "A_log"] = rnd(H, std=0.5) - 1.0
            w[q + "norm"] = 1.0 + rnd(e, std=0.2)
            w[q + "a1"], w[q + "a2"] = lin(ra, W), lin(H * d, ra, 1.5)
            w[q + "dt_bias"] = rnd(H * d, std=0.7) - 1.0
            w[q + "g1"], w[q + "g2"] = lin(rg, W), lin(H * e, rg, 2.0)
            w[q + "o"] = lin(W, H * e, 2.0)
        else:
            H, P, N, G, K = m["heads"], m["vdim"], m["state"], m.get("groups", 1), m["conv"]
            inner, ch = H * P, H * P + 2 * G * N
            w[q + "in"] = lin(2 * inner + 2 * G * N + H, W, 1.5)
            w[q + "conv"], w[q + "conv.b"] = rnd(ch, K, std=0.6), rnd(ch, std=0.2)
            w[q + "dt_bias"] = rnd(H, std=0.5) - 0.5
            w[q + "A_log"] = rnd(H, std=0.5) - 0.5
            w[q + "D"] = 1.0 + rnd(H, std=0.3)
            w[q + "norm"] = 1.0 + rnd(inner, std=0.2)
            w[q + "o"] = lin(W, inner, 1.5)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write_folder(folder: str, cfg: dict, weights: Dict[str, torch.Tensor]) -> str:
    """``config.json`` and ``model.safetensors`` (8-byte length, JSON header, data) written by hand."""
    import struct
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, t in weights.items():
        raw = t.contiguous().view(torch.int16).numpy().tobytes() if t.dim() else \
            t.reshape(1).view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    return folder


def random_requests(cfg: dict, lengths: List[int], seed: int) -> Dict[str, List[int]]:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
