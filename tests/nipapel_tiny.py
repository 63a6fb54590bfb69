"""Tiny Nipapel configurations and weights for the tests.

The configurations differ from one another in every size and option: order and kinds of layers, layers
without a feed-forward, dense and routed feed-forwards, one expert per token and all experts per token, key and
value sizes that differ, one head, as many key heads as heads or fewer, windows of 1, 5, 9 and more than a
prompt, no kept first tokens, more kept first tokens than a window or a page holds, rotation of part of a head,
all of it or none, layers that borrow latents from a layer whose window is narrower or wider than theirs.
Weights are drawn so that scores and activations stay of order one (a model whose mixers put out almost nothing
hides their faults) and are rounded to bfloat16, so that both precision paths and the plain model read the same
numbers.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List

import torch


def _attn(heads, kv, dim, vdim, window, keep=None, rot=None, scale=None):
    mask = {"size": window}
    if keep is not None:
        mask["keep_first"] = keep
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": mask,
         "scale": scale if scale is not None else dim ** -0.5}
    if rot:
        m["rot"] = rot
    return m


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base=10000.0, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim},
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, limit, experts, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


CONFIG_A = {
    "architecture": "Nipapel", "vocab": 101, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mlp": _dense(80, 1.0),
         "mixer": _attn(4, 2, 16, 8, 9, keep=3, rot={"base": 10000.0, "dims": 8}, scale=0.3)},
        {"type": "latent_attention", "mlp": _moe(40, 0.7, 5, 2), "mixer": _latent(3, 8, 4, 12, 20, 24, 7, base=100.0)},
        {"type": "latent_attention", "mlp": None, "mixer": _latent(2, 12, 4, 8, 20, 16, 13, base=100.0, kv_from=1)},
        {"type": "attention", "mlp": _moe(24, 2.5, 3, 1),
         "mixer": _attn(2, 2, 12, 20, 33, rot={"base": 500.0, "dims": 12})},
    ],
}

CONFIG_B = {
    "architecture": "Nipapel", "vocab": 131, "width": 72, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mlp": _dense(96, 3.0), "mixer": _latent(5, 16, 8, 16, 24, 40, 64, base=50.0)},
        {"type": "attention", "mlp": _moe(56, 1.2, 4, 4), "mixer": _attn(6, 1, 24, 40, 5, keep=9, scale=0.25)},
        {"type": "latent_attention", "mlp": _moe(32, 0.9, 6, 3),
         "mixer": _latent(1, 20, 8, 28, 24, 12, 3, base=50.0, kv_from=0)},
        {"type": "latent_attention", "mlp": None, "mixer": _latent(4, 4, 2, 6, 10, 8, 1)},
        {"type": "attention", "mlp": None, "mixer": _attn(1, 1, 20, 96, 1, keep=1, rot={"base": 30.0, "dims": 2})},
    ],
}

# shapes that the bfloat16 path takes to the tensor cores (value or latent size 64 or 128, key rows a multiple of
# 16), once with more heads than one block finishes; expert sizes that the tensor-core grouped product takes
CONFIG_C = {
    "architecture": "Nipapel", "vocab": 160, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mlp": _moe(64, 1.5, 4, 2),
         "mixer": _attn(4, 2, 32, 64, 40, keep=4, rot={"base": 10000.0, "dims": 16})},
        {"type": "latent_attention", "mlp": _dense(128, 2.0), "mixer": _latent(4, 16, 16, 16, 64, 32, 24)},
        {"type": "latent_attention", "mlp": _moe(64, 1.0, 8, 3), "mixer": _latent(6, 8, 16, 24, 64, 48, 50, kv_from=1)},
        {"type": "attention", "mlp": None, "mixer": _attn(36, 4, 16, 64, 23, keep=1)},
        {"type": "latent_attention", "mlp": _dense(64, 1.0), "mixer": _latent(8, 32, 32, 16, 128, 64, 17, base=1000.0)},
    ],
}

# one of everything that a model may happen to make equal or one
CONFIG_D = {
    "architecture": "Nipapel", "vocab": 64, "width": 40, "norm": {"eps": 3e-6},
    "layers": [
        {"type": "attention", "mlp": _moe(16, 0.5, 1, 1), "mixer": _attn(1, 1, 8, 8, 1, keep=0)},
        {"type": "latent_attention", "mlp": _dense(48, 0.8), "mixer": _latent(1, 8, 2, 8, 8, 8, 200)},
        {"type": "attention", "mlp": _dense(48, 6.0),
         "mixer": _attn(5, 5, 10, 6, 300, keep=2, rot={"base": 1000.0, "dims": 4})},
    ],
}

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D}


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """``name -> bfloat16 tensor`` for every tensor the configuration implies (names built here from the
    configuration alone, so the engine's own manifest is checked against an independent one)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def rnd(*shape, std=1.0):
        return torch.randn(*shape, generator=g) * std

    def lin(out, inn, gain=1.0):
        return rnd(out, inn, std=gain / math.sqrt(inn))

    w: Dict[str, torch.Tensor] = {"embed": rnd(cfg["vocab"], W), "embed.norm": rnd(W, std=0.2),
                                  "head": lin(cfg["vocab"], W, 2.0), "final.norm": rnd(W, std=0.2)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = rnd(W, std=0.2)
        q = p + "mix."
        if L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * d, W), lin(G * d, W), lin(G * e, W, 1.5)
            w[q + "q.norm"], w[q + "k.norm"] = 1.5 + rnd(d, std=0.3), 1.5 + rnd(d, std=0.3)
            w[q + "o"] = lin(W, H * e, 1.5)
        else:
            H, d, r, e, c, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w[q + "dq"], w[q + "dq.norm"] = lin(qr, W), 1.0 + rnd(qr, std=0.2)
            w[q + "uq"] = lin(H * (d + r), qr, 2.0)
            if m.get("kv_from") is None:
                w[q + "dkv"], w[q + "dkv.norm"] = lin(c + r, W, 1.5), 1.0 + rnd(c, std=0.2)
            w[q + "uk"], w[q + "uv"] = lin(H * d, c, 2.0), lin(H * e, c, 1.5)
            w[q + "g"], w[q + "o"] = lin(H * e, W, 2.0), lin(W, H * e, 2.0)
        mlp = L.get("mlp")
        q = p + "mlp."
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            w[q + "gate"], w[q + "up"], w[q + "down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
        else:
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            w[q + "router"], w[q + "router.b"] = lin(E, W, 2.0), rnd(E, std=0.5)
            for x in range(E):
                w[f"{q}e{x}.gate"], w[f"{q}e{x}.up"], w[f"{q}e{x}.down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff, 1.5)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write_folder(folder: str, cfg: dict, weights: Dict[str, torch.Tensor]) -> str:
    """``config.json`` and ``model.safetensors`` (8-byte length, JSON header, data) written by hand."""
    import struct
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, t in weights.items():
        raw = t.contiguous().view(torch.int16).numpy().tobytes()
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
