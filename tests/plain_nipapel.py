"""A plain, slow Nipapel in PyTorch on the CPU: one function per mechanism, whole sequences at once, no
cache carried between calls.  It shares no code with the engine and is what the engine's kernels, parts and
step function are compared with.  ``dtype`` float64 gives an oracle whose own rounding is far below the
float32 engine's.

Notation: ``T`` tokens, ``W`` width, ``H`` query heads, ``G`` key/value heads, ``d`` key size, ``e`` value
size, ``r`` rotated size, ``c`` latent size.  Weights are a dict ``name -> tensor`` with the checkpoint's
names; a configuration is the dictionary of ``config.json``.
"""

from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch


def same(t):
    return t


def as_bfloat16(t):
    """Round to bfloat16 and back: handed to ``forward`` as ``rnd`` it rounds where the engine's bfloat16
    path stores 16 bits (the inputs of its matrix products and the cache)."""
    return t.to(torch.bfloat16).to(t.dtype)


# --------------------------------------------------------------------------- #
# norms
# --------------------------------------------------------------------------- #

def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The checkpoint holds the gain's offset from one: the gain is ``1 + w``."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


# --------------------------------------------------------------------------- #
# rotations
# --------------------------------------------------------------------------- #

def _angles(T: int, dims: int, base: float, dtype, first_position: int = 0):
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    p = torch.arange(first_position, first_position + T, dtype=torch.float64)
    a = p[:, None] * f[None, :]
    return torch.cos(a).to(dtype), torch.sin(a).to(dtype)


def rotate_halves(x, dims: int, base: float):
    """``x [T, heads, d]``: coordinate ``i`` of the first ``dims`` is paired with ``i + dims/2``."""
    T = x.shape[0]
    cos, sin = _angles(T, dims, base, x.dtype)
    h = dims // 2
    u, v = x[..., :h], x[..., h:dims]
    cu = cos[:, None, :]
    su = sin[:, None, :]
    out = x.clone()
    out[..., :h] = u * cu - v * su
    out[..., h:dims] = v * cu + u * su
    return out


def rotate_neighbours(x, dims: int, base: float):
    """``x [T, heads, d]``: coordinate ``2i`` of the first ``dims`` is paired with ``2i + 1``."""
    T = x.shape[0]
    cos, sin = _angles(T, dims, base, x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    cu = cos[:, None, :]
    su = sin[:, None, :]
    out = x.clone()
    out[..., 0:dims:2] = u * cu - v * su
    out[..., 1:dims:2] = v * cu + u * su
    return out


# --------------------------------------------------------------------------- #
# masks and the softmax over visible keys
# --------------------------------------------------------------------------- #

def visible(T: int, size: int, keep_first: int = 0) -> torch.Tensor:
    """``[T, T]`` bool: query ``i`` sees key ``j`` iff ``j <= i`` and (``i - j < size`` or ``j < keep_first``)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def masked_softmax_attention(q, k, v, scale: float, mask: torch.Tensor):
    """``q [T, H, d]``, ``k [T, G, d]``, ``v [T, G, e]`` -> ``[T, H, e]``; head ``h`` reads key/value head
    ``h // (H / G)``."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = []
    for h in range(H):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out.append(p @ v[:, g, :])
    return torch.stack(out, dim=1)


# --------------------------------------------------------------------------- #
# mixers
# --------------------------------------------------------------------------- #

def attention_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, rnd: Callable = same):
    """Grouped-query attention: per-head unit-RMS queries and keys with a shared gain, rotation of part of
    each head by halves, a window of recent keys plus the first keys of the sequence."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, e)
    q = norm_plain(q, w[p + "q.norm"], eps)
    k = norm_plain(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate_halves(q, rot["dims"], rot["base"])
        k = rotate_halves(k, rot["dims"], rot["base"])
    mask = visible(T, m["mask"]["size"], m["mask"].get("keep_first", 0))
    a = masked_softmax_attention(rnd(q), rnd(k), rnd(v), m["scale"], mask)
    return rnd(a).reshape(T, H * e) @ w[p + "o"].T


def latent_of(h, w, p: str, m: dict, eps: float, rnd: Callable = same):
    """What a latent-attention layer keeps per token: the normalised latent ``[T, c]`` and the rotated key
    part that all heads share ``[T, r]``."""
    T = h.shape[0]
    c, r = m["kv_rank"], m["rot_dim"]
    dkv = h @ w[p + "dkv"].T
    lat = norm_plain(dkv[:, :c], w[p + "dkv.norm"], eps)
    kr = rotate_neighbours(dkv[:, c:].reshape(T, 1, r), r, m["rot"]["base"]).reshape(T, r)
    return rnd(lat), rnd(kr)


def latent_attention_mixer(h, w, p: str, m: dict, eps: float, kept, rnd: Callable = same):
    """Attention through latents.  ``kept`` is ``(latent [T, c], rotated key part [T, r])`` of this layer or
    of the layer it borrows them from."""
    T = h.shape[0]
    H, d, r, e = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    lat, kr = kept
    cq = norm_plain(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (rnd(cq) @ w[p + "uq"].T).view(T, H, d + r)
    q_plain = q[..., :d]
    q_rot = rotate_neighbours(q[..., d:], r, m["rot"]["base"])
    k_plain = (lat @ w[p + "uk"].T).view(T, H, d)
    v = (lat @ w[p + "uv"].T).view(T, H, e)
    qq = torch.cat([q_plain, q_rot], dim=-1)
    kk = torch.cat([k_plain, kr[:, None, :].expand(T, H, r)], dim=-1)
    mask = visible(T, m["mask"]["size"], 0)
    a = masked_softmax_attention(qq, kk, v, m["scale"], mask)
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return rnd(a.reshape(T, H * e) * gate) @ w[p + "o"].T


# --------------------------------------------------------------------------- #
# feed-forward
# --------------------------------------------------------------------------- #

SWISH_SLOPE = 1.702


def clamped_glu(g, u, limit: float):
    """``g`` capped from above, ``u`` clamped on both sides; ``g * sigmoid(1.702 g) * (u + 1)``."""
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, min=-limit, max=limit)
    return g * torch.sigmoid(SWISH_SLOPE * g) * (u + 1.0)


def gated_ff(h, w_gate, w_up, w_down, limit: float, rnd: Callable = same):
    return rnd(clamped_glu(h @ w_gate.T, h @ w_up.T, limit)) @ w_down.T


def routed_ff(h, w, p: str, mlp: dict, rnd: Callable = same, chosen: Optional[list] = None, forced=None):
    """The ``top`` experts with the largest router logits (weight times input plus bias); their weights are
    the softmax over the chosen logits alone.  ``chosen`` receives ``(indices, logits)``; ``forced``
    (``[T, top]``) replaces the choice (the weights are then the softmax over the forced experts' logits)."""
    E, K = mlp["router"]["experts"], mlp["router"]["top"]
    limit = mlp["expert"]["limit"]
    z = h.to(torch.float64) @ w[p + "router"].to(torch.float64).T + w[p + "router.b"].to(torch.float64)
    picked = torch.topk(z, K, dim=-1).indices if forced is None else forced
    if chosen is not None:
        chosen.append((picked, z))
    gate = torch.softmax(z.gather(1, picked), dim=-1).to(h.dtype)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for slot in range(K):
            e = int(picked[t, slot])
            q = f"{p}e{e}."
            out[t] += gate[t, slot] * gated_ff(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"], limit, rnd)[0]
    return out


def feed_forward(h, w, p: str, mlp: Optional[dict], rnd: Callable = same, chosen: Optional[list] = None,
                 forced=None):
    if mlp is None:
        return torch.zeros_like(h)
    if mlp["kind"] == "dense":
        return gated_ff(h, w[p + "gate"], w[p + "up"], w[p + "down"], mlp["limit"], rnd)
    return routed_ff(h, w, p, mlp, rnd, chosen, forced)


# --------------------------------------------------------------------------- #
# the model
# --------------------------------------------------------------------------- #

def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            rnd: Callable = same, layers_out: Optional[list] = None, chosen: Optional[dict] = None,
            forced: Optional[dict] = None):
    """Logits ``[T, vocab]`` of a whole sequence.  ``layers_out`` receives the residual stream after every
    layer; ``chosen[layer]`` the ``(experts, router logits)`` of every routed layer; ``forced[layer]``
    (``[T, top]``) overrides a routed layer's choice."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = norm_one_plus(x, w["embed.norm"], eps)
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rnd(norm_one_plus(x, w[p + "norm1"], eps))
        if layer["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", m, eps, rnd)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_of(h, w, p + "mix.", m, eps, rnd)
                src = i
            y = latent_attention_mixer(h, w, p + "mix.", m, eps, kept[src], rnd)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        rec = [] if chosen is not None else None
        x = x + (y + feed_forward(h, w, p + "mlp.", layer.get("mlp"), rnd, rec,
                                  None if forced is None else forced.get(i)))
        if rec:
            chosen[i] = rec[0]
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rnd(norm_one_plus(x, w["final.norm"], eps))
    return x @ w["head"].T


def greedy(config: dict, weights, prompt: List[int], n: int, dtype=torch.float64) -> List[int]:
    """``n`` tokens, each the arg-max of the logits at the last position of all tokens so far."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(config, weights, toks, dtype)[-1])))
    return toks[len(prompt):]
