"""Attention through a latent: per token the cache holds ONE row that all heads share.

With ``h`` the layer's input, ``c_q = norm(W_dq h)`` and ``q_h = W_uq,h c_q = [q_h^plain | q_h^rot]`` per head;
``[c | k^rot] = W_dkv h`` with ``c`` brought to unit root mean square (times a gain) and ``k^rot`` rotated by
position; key and value of head ``h`` are ``W_uk,h c`` and ``W_uv,h c``;
``score = (q_h^plain . W_uk,h c + rot(q_h^rot) . rot(k^rot)) * scale``; softmax over a window of keys; the
heads' outputs times ``sigmoid(W_g h)``; then ``W_o``.

Only ``[c | rot(k^rot)]`` is cached (``LatentNeed``).  The key matrices are folded into the queries,
``q_h' = W_uk,h^T q_h^plain`` (so ``q_h^plain . W_uk,h c = q_h' . c``), and the value matrices are applied
after the weighted sum (``sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j``): the attention itself then runs over
one shared key/value head whose keys are the cached rows and whose values are their first ``kv_rank``
numbers, with the engine's attention kernels, for prompts and for decoding alike: the float32 path takes
``ops.functional.attention_mix`` for every step; the bfloat16 path takes ``attention_mix_tc`` (split over the
keys) for decode steps and, for prompt portions, the tcgen05 kernel with (query, head) pairs as the rows of a
query tile (``prefill_attention_tc_shared``) where the sizes allow, else ``attention_mix_tc``.  A layer may read
the rows another layer caches (``shares_cache``): it then has no ``W_dkv`` of its own.

The rotation pairs neighbouring dimensions (``2i`` with ``2i + 1``).
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from ..ops import functional as F
from .base import CacheBinding, LatentNeed, Mixer, Runtime, StepContext, TensorDecl, linear


class LatentAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim`` (unrotated query/key size per head), ``rot_dim``
    (rotated size), ``value_dim``, ``kv_rank``, ``q_rank``, ``window`` (0 = all keys), ``scale``, ``eps`` (of
    the two latent norms), ``position`` (a ``PartSpec`` of category ``position`` whose table has
    ``rot_dim / 2`` frequencies), ``shares_cache`` (reads another layer's cached rows; no ``dkv`` tensors).

    Tensors below the prefix: ``dq [q_rank, hidden]``, ``dq.norm [q_rank]``, ``uq [heads*(head_dim+rot_dim),
    q_rank]``, ``dkv [kv_rank+rot_dim, hidden]``, ``dkv.norm [kv_rank]``, ``uk [heads*head_dim, kv_rank]``,
    ``uv [heads*value_dim, kv_rank]``, ``g [heads*value_dim, hidden]``, ``o [hidden, heads*value_dim]``."""

    graph_safe = True
    kernel_files = ("attention_latent.cu", "attention_mix.cu", "attention_mix_tc.cu", "attention_prefill_tc.cu",
                    "dense_f32.cu", "elementwise.cu")

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = self.params
        self.W = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.d = int(p["head_dim"])
        self.r = int(p["rot_dim"])
        self.e = int(p["value_dim"])
        self.c = int(p["kv_rank"])
        self.qr = int(p["q_rank"])
        self.window = int(p.get("window", 0))
        self.scale = float(p.get("scale", (self.d + self.r) ** -0.5))
        self.eps = float(p["eps"])
        self.shares_cache = bool(p.get("shares_cache", False))
        pos: PartSpec = p.get("position") or PartSpec("none")
        self.position = part_class("position", pos.kind)(pos.params, prefix)
        if self.r % 2:
            raise ValueError(f"latent attention: the rotated part ({self.r}) must be even")

    def tensor_decls(self) -> List[TensorDecl]:
        p = self.prefix
        out = [TensorDecl(p + "dq", (self.qr, self.W)), TensorDecl(p + "dq.norm", (self.qr,), "norm"),
               TensorDecl(p + "uq", (self.nh * (self.d + self.r), self.qr))]
        if not self.shares_cache:
            out += [TensorDecl(p + "dkv", (self.c + self.r, self.W)), TensorDecl(p + "dkv.norm", (self.c,), "norm")]
        out += [TensorDecl(p + "uk", (self.nh * self.d, self.c)), TensorDecl(p + "uv", (self.nh * self.e, self.c)),
                TensorDecl(p + "g", (self.nh * self.e, self.W)), TensorDecl(p + "o", (self.W, self.nh * self.e))]
        return out

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        m, dev, p = rt.precision.matrix, rt.device, self.prefix
        f32 = lambda t: t.to(device=dev, dtype=torch.float32).contiguous()      # norms are float arithmetic
        self.w_dq = m(tensors[p + "dq"], dev)
        self.dq_gain = f32(tensors[p + "dq.norm"])
        self.w_uq = m(tensors[p + "uq"], dev)
        # the gate and (unless the rows come from another layer) the latent in one product of the input
        rows = [m(tensors[p + "g"], dev)]
        self.dkv_gain = None
        if not self.shares_cache:
            rows.append(m(tensors[p + "dkv"], dev))
            self.dkv_gain = f32(tensors[p + "dkv.norm"])
        self.w_g_dkv = torch.cat(rows, dim=0).contiguous()
        uk = m(tensors[p + "uk"], dev).view(self.nh, self.d, self.c)
        uv = m(tensors[p + "uv"], dev).view(self.nh, self.e, self.c)
        if rt.act == torch.float32:
            self.w_uk_fold = uk.transpose(1, 2).contiguous()         # [H, c, d]: q' = w . q_plain
            self.w_uv = uv.contiguous()                              # [H, e, c]
        else:
            self.w_uk_fold = uk.contiguous()                         # [H, d, c] as the right operand of bmm
            self.w_uv = uv.transpose(1, 2).contiguous()              # [H, c, e]
        self.w_o = m(tensors[p + "o"], dev)
        self.inv_freq = self.position.table(dev)
        if self.r and (self.inv_freq is None or self.inv_freq.numel() != self.r // 2):
            raise ValueError(f"latent attention: a rotated part of {self.r} needs {self.r // 2} frequencies")
        dk = self.c + self.r
        if not F.attention_mix_supported(self.nh, 1, dk, self.c, rt.act):
            raise ValueError(f"latent attention: {self.nh} heads over rows of {dk} with values of {self.c} "
                             f"are more than one block of the kernel holds")
        self._tensor_cores = rt.act == torch.bfloat16 and F.attention_mix_tc_supported(self.nh, 1, dk, self.c)
        # prompt portions on the tensor-memory attention: its blocks want whole SMs (a block arrangement that
        # runs another part beside this one asks)
        self.large_steps_fill_the_device = self._tensor_cores

    def prefetch_first(self, ctx: StepContext, cache: Optional[CacheBinding]) -> None:
        F.l2_prefetch(self.w_dq)
        F.l2_prefetch(self.w_g_dkv)

    def cache_need(self):
        return LatentNeed(self.c, self.r, self.window)

    def _span(self, max_kv_len: int) -> int:
        return min(self.window, max_kv_len) if self.window > 0 else max_kv_len

    def scratch_need(self, max_requests: int, max_context: int) -> Dict[str, int]:
        splits = F.attention_mix_tc_splits(self._span(max_context))
        return {"attn_mix_part_o": max_requests * splits * self.nh * self.c,
                "attn_mix_part_ml": max_requests * splits * self.nh * 2}

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        view = ctx.kv_groups[cache.group]
        rows = view.tensors["latent"][cache.layer_slot]              # [pages, 1, page_size, c + r]
        T, H, d, r, e, c = ctx.num_tokens, self.nh, self.d, self.r, self.e, self.c
        f32 = self.rt.act == torch.float32
        # queries through their latent
        cq = F.add_rmsnorm(linear(x, self.w_dq, torch.float32), None, self.dq_gain, self.eps, self.rt.act)
        q = linear(cq, self.w_uq, torch.float32)
        # gate, and this token's cached row
        gk = linear(x, self.w_g_dkv, torch.float32)
        if not self.shares_cache:
            if not cache.writes:
                raise RuntimeError("latent attention: a layer with a latent projection of its own must own its cache")
            F.latent_store(gk, H * e, ctx.positions, self.inv_freq, self.dkv_gain, self.eps, view.slot_mapping, rows,
                           c, r)
        q_full, q_plain = F.latent_query(q, ctx.positions, self.inv_freq, H, d, r, c, self.rt.act, not f32)
        if f32:
            F.dense_f32_heads(q, self.w_uk_fold, out=q_full, x_head_stride=d + r, out_head_stride=c + r)
        else:
            # written head by head into its place before the rotated parts (rows H * (c + r) apart)
            torch.bmm(q_plain.transpose(0, 1), self.w_uk_fold, out=q_full.transpose(0, 1)[:, :, :c])
        # one shared key/value head: keys are the cached rows, values their first c numbers
        if not self._tensor_cores:
            a = F.attention_mix(q_full, rows, rows, None, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len,
                                self.window, self.scale, 0.0, value_dim=c)
        elif ctx.all_decode and "attn_mix_part_o" in ctx.scratch:
            splits = F.attention_mix_tc_splits(self._span(ctx.max_kv_len))
            a = F.attention_mix_tc(q_full, rows, rows, None, view.block_table, ctx.q_start, ctx.kv_len, 1, self.window,
                                   self.scale, 0.0, splits, ctx.scratch["attn_mix_part_o"],
                                   ctx.scratch["attn_mix_part_ml"], value_dim=c)
        elif F.prefill_attention_tc_shared_supported(H, c + r, c, view.page_size):
            # prompt portions (and what decodes beside them): the tensor-memory attention with (query, head)
            # pairs as the rows of a tile
            a = F.prefill_attention_tc_shared(q_full, rows, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len,
                                              self.window, self.scale, c)
        else:
            a = F.attention_mix_tc(q_full, rows, rows, None, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len,
                                   self.window, self.scale, 0.0, value_dim=c)
        # values of the heads from the weighted latents, gate, output
        if f32:
            v = F.dense_f32_heads(a.view(T, H * c), self.w_uv)
            gated = F.sigmoid_gate(v, False, gk, 0, H, e)
        else:
            v = torch.bmm(a.transpose(0, 1), self.w_uv)              # [H, T, e]
            gated = F.sigmoid_gate(v, True, gk, 0, H, e)
        return linear(gated, self.w_o, torch.float32)


register_part("mixer", "latent_attention", LatentAttention)
