"""A plain, slow Vizalix in PyTorch on the CPU: one function per mechanism, whole sequences at once,
no cache, no state carried between calls.  It shares no code with the engine and is what the engine's
kernels, parts and step function are compared with.  ``dtype`` float64 gives an oracle whose own rounding
is far below the float32 engine's.

Notation: ``T`` tokens, ``W`` width, ``H`` heads, ``G`` key/value (or B/C) heads, ``d`` key size, ``e`` value
size, ``N`` state size.  Weights are a dict ``name -> tensor`` with the checkpoint's names.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, gain, eps):
    return unit_rms(x, eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.logaddexp(z, torch.zeros_like(z))


def short_conv_silu(x, taps_w, bias=None):
    """``x [T, C]``, ``taps_w [C, K]``: ``y_t = sum_j taps_w[:, j] * x_(t-(K-1-j))`` with zeros before the
    sequence, plus ``bias``, then silu."""
    T, C = x.shape
    K = taps_w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            s = t - (K - 1 - j)
            if s >= 0:
                y[t] = y[t] + taps_w[:, j] * x[s]
    if bias is not None:
        y = y + bias
    return silu(y)


def same(t):
    return t


def as_bfloat16(t):
    """Round to bfloat16 and back: handed to ``forward`` as ``rnd`` it rounds where the engine's bfloat16 path
    stores activations in 16 bits (the inputs of its matrix products), so that what is left between the two
    is the order of additions and not the model's own sensitivity to rounding."""
    return t.to(torch.bfloat16).to(t.dtype)


def gated_mlp(x, w_gate, w_up, w_down, rnd=same):
    return rnd(gelu_tanh(rnd(x @ w_gate.T)) * rnd(x @ w_up.T)) @ w_down.T


def delta_rule(q, k, v, beta, decay):
    """``q, k [T, G, d]`` (already unit vectors, q scaled), ``v [T, H, e]``, ``beta [T, H]``,
    ``decay [T, H, d]``.  Returns ``o [T, H, e]``."""
    T, H, e = v.shape
    G, d = q.shape[1], q.shape[2]
    out = torch.zeros(T, H, e, dtype=v.dtype)
    for h in range(H):
        kh = h // (H // G)
        S = torch.zeros(d, e, dtype=v.dtype)
        for t in range(T):
            S = decay[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, kh])
            S = S + k[t, kh][:, None] * u[None, :]
            out[t, h] = S.T @ q[t, kh]
    return out


def channel_delta_mixer(x, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, rnd=same):
    T = x.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(x @ w[p + "q"].T, w[p + "q.conv"]).view(T, G, d)
    k = short_conv_silu(x @ w[p + "k"].T, w[p + "k.conv"]).view(T, G, d)
    v = short_conv_silu(x @ w[p + "v"].T, w[p + "v.conv"]).view(T, H, e)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(x @ w[p + "b"].T)
    a = rnd(x @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(a).view(T, H, d))
    o = delta_rule(q, k, v, beta, decay)
    gate = torch.sigmoid(rnd(x @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, e)
    o = unit_rms(o, eps) * w[p + "norm"] * gate
    return rnd(o).reshape(T, H * e) @ w[p + "o"].T


def rotary_frequencies(rot: dict) -> torch.Tensor:
    D = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / D) for i in range(D // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f.tolist():
            wavelength = 2.0 * math.pi / fi
            if wavelength < sc["original"] / sc["high"]:
                out.append(fi)
            elif wavelength > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f


def rotate(x, positions, rot: Optional[dict]):
    """``x [T, heads, d]``: the first ``dims`` dimensions rotated in pairs ``(i, i + dims/2)``."""
    if not rot:
        return x
    D = rot["dims"]
    ang = positions.to(torch.float64)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    lo, hi, rest = x[..., :D // 2], x[..., D // 2:D], x[..., D:]
    return torch.cat([lo * c - hi * s, hi * c + lo * s, rest], dim=-1)


def mixed_head_attention(q, k, v, scale, cap, talk, window):
    """``q [T, H, d]``, ``k [T, G, d]``, ``v [T, G, e]``: scores scaled, capped, mixed over the heads with
    ``talk [H, H]`` (or None), masked to ``0 <= i - j < window``, softmax, times v."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    scores = torch.stack([q[:, h] @ k[:, h // rep].T for h in range(H)]) * scale          # [H, T, T]
    if cap:
        scores = cap * torch.tanh(scores / cap)
    if talk is not None:
        scores = torch.einsum("hg,gij->hij", talk, scores)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = (i - j >= 0) & (i - j < window)
    scores = scores.masked_fill(~visible, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.stack([probs[h] @ v[:, h // rep] for h in range(H)], dim=1)              # [T, H, e]


def attention_mixer(x, w, p, m, eps, rnd=same):
    T = x.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rnd(rotate((x @ w[p + "q"].T).view(T, H, d), pos, m.get("rot")))
    k = rnd(rotate((x @ w[p + "k"].T).view(T, G, d), pos, m.get("rot")))
    v = rnd((x @ w[p + "v"].T).view(T, G, e))
    o = mixed_head_attention(q, k, v, m["scale"], m.get("softcap"), w.get(p + "talk"), m["mask"]["size"])
    return rnd(o).reshape(T, H * e) @ w[p + "o"].T


def state_space_scan(xh, B, C, dt, A, D):
    """``xh [T, H, P]``, ``B, C [T, G, N]``, ``dt [T, H]`` (after softplus), ``A, D [H]``."""
    T, H, P = xh.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(xh)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros(N, P, dtype=xh.dtype)
        for t in range(T):
            S = torch.exp(-A[h] * dt[t, h]) * S + dt[t, h] * B[t, g][:, None] * xh[t, h][None, :]
            y[t, h] = S.T @ C[t, g] + D[h] * xh[t, h]
    return y


def mamba2_mixer(x, w, p, m, eps, rnd=same):
    T = x.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    inner = H * P
    z, xbc, dt = torch.split(x @ w[p + "in"].T, [inner, inner + 2 * G * N, H], dim=-1)
    xbc = short_conv_silu(xbc, w[p + "conv"], w[p + "conv.b"])
    xh, B, C = torch.split(xbc, [inner, G * N, G * N], dim=-1)
    dt = softplus(dt + w[p + "dt_bias"])
    y = state_space_scan(xh.reshape(T, H, P), B.reshape(T, G, N), C.reshape(T, G, N), dt,
                         torch.exp(w[p + "A_log"]), w[p + "D"])
    y = y.reshape(T, inner) * silu(z)
    ng = m.get("norm_groups", 1)
    y = unit_rms(y.view(T, ng, inner // ng), eps).reshape(T, inner) * w[p + "norm"]
    return rnd(y) @ w[p + "o"].T


MIXERS = {"channel_delta": channel_delta_mixer, "attention": attention_mixer, "mamba2": mamba2_mixer}


def layer_runs(cfg: dict) -> List[tuple]:
    """``(layer, pass it opens or None)`` in running order."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            residuals: Optional[list] = None, rnd=same) -> torch.Tensor:
    """Logits ``[T, vocab]`` of the whole sequence; ``residuals`` collects the stream after every layer run;
    ``rnd`` is applied to every input of a matrix product (see :func:`as_bfloat16`)."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    x0 = x
    for i, opens in layer_runs(cfg):
        if opens is not None:
            x = rnd(torch.cat([x, x0], dim=-1)) @ w["loop.in"].T + w["loop.step"][opens]
        L, p = cfg["layers"][i], f"l{i}."
        delta = MIXERS[L["type"]](rnd(scalar_norm(x, w[p + "norm1"], eps)), w, p + "mix.", L["mixer"], eps, rnd)
        if L.get("mlp"):
            delta = delta + gated_mlp(rnd(scalar_norm(x, w[p + "norm2"], eps)), w[p + "mlp.gate"], w[p + "mlp.up"],
                                      w[p + "mlp.down"], rnd)
        x = x + delta
        if residuals is not None:
            residuals.append(x.clone())
    return rnd(scalar_norm(x, w["final.norm"], eps)) @ w["head"].T


def greedy(cfg, weights, prompt: List[int], new_tokens: int, dtype=torch.float64) -> List[int]:
    toks = list(prompt)
    out = []
    for _ in range(new_tokens):
        nxt = int(torch.argmax(forward(cfg, weights, toks, dtype)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
