"""Grouped-query attention over the paged cache (atom/models/qwen3.py:59-163).

   qkv = x W_qkv^T (+ b);  q, k, v = split(qkv, [nh*hd, nkv*hd, nkv*hd])          (:146-147)
   q_h = RMSNorm_hd(q_h; w_q),  k_g = RMSNorm_hd(k_g; w_k)   per head, if qk_norm   (:159-160)
   q, k rotated by the position encoding; k, v written to the request's pages
   o_t = softmax_j(scale * q_t . k_j) v_j  over j <= pos(t) (and j > pos(t) - window)
   y = o W_o^T                                                                      (:162)
scale = hd^-0.5 (:88) unless given.  Query head h reads kv head h // (nh / nkv).
One kernel semantics serves prompt portions and decoded tokens: every token attends to
the keys of its own request that lie in the cache after this step's write.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import native
from . import registry
from .base import Mixer, PositionEncoding
from .linear import PendingProduct, linear, may_defer
from .registry import register
from .spec import CacheNeed, ParamSpec, PartSpec


@register("mixer", "paged_attention")
class PagedAttention(Mixer):
    takes_scaled_rows = True      # x may be ScaledRows: the qkv product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the output projection on unrun

    @property
    def graph_safe(self) -> bool:      # its own launches are; the position encoding answers for itself
        return self.position.graph_safe

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, qk_norm: bool = False, norm_eps: float = 0.0,
                 bias: bool = False, window: Optional[int] = None, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size, self.nh, self.nkv, self.hd = hidden_size, num_heads, num_kv_heads, head_dim
        self.qk_norm, self.norm_eps, self.bias, self.window = qk_norm, norm_eps, bias, window
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.position = registry.build("position", position)
        self._table = None
        self._long_rows = None    # packed rows from which a request runs on the tcgen05 kernel (0: never)

    def params(self) -> Dict[str, ParamSpec]:
        q, kv = self.nh * self.hd, self.nkv * self.hd
        p = {
            "qkv.weight": ParamSpec((q + 2 * kv, self.hidden_size), rows=(q, kv, kv)),
            "o.weight": ParamSpec((self.hidden_size, q)),
        }
        if self.bias:
            p["qkv.bias"] = ParamSpec((q + 2 * kv,), role="vector", init="zeros", rows=(q, kv, kv))
        if self.qk_norm:
            p["q_norm.weight"] = ParamSpec((self.hd,), role="vector", init="norm")
            p["k_norm.weight"] = ParamSpec((self.hd,), role="vector", init="norm")
        return p

    def cache_need(self) -> CacheNeed:
        return CacheNeed("pages", num_kv_heads=self.nkv, head_dim=self.hd, window=self.window)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self._table = self.position.table(rt)
        self._check_sizes()

    def _check_sizes(self) -> None:
        if self.hd > 512:
            raise ValueError(f"paged_attention: head_dim {self.hd} is beyond what the kernels take (512)")

    def forward(self, x, step, cache, writes_cache, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        nh, nkv, hd = self.nh, self.nkv, self.hd
        qkv = linear(x, self.w_qkv_weight, getattr(self, "w_qkv_bias", None),
                     ws.get("attn.qkv", (T, (nh + 2 * nkv) * hd), dt))
        bt = step.block_tables[cache.group]
        qw = self.w_q_norm_weight if self.qk_norm else None
        kw = self.w_k_norm_weight if self.qk_norm else None
        kp = cache.k_pages if writes_cache else None
        vp = cache.v_pages if writes_cache else None
        o = ws.get("attn.o", (T, nh * hd), dt)
        if self._rotates_in_decode(step, cache):
            # a decode step: norm, rotation and cache write are the attention kernel's own prologue
            plan = self.launch_plan(step)
            scratch = None
            if plan[2] > 1:
                scratch = ws.get("attn.splits", (native.flash_scratch_elems(T, nh, hd, plan[2]),), torch.float32)
            native.flash_attention_rotating(
                o, qkv, cache.k_pages, cache.v_pages, bt, step.cu_q, step.ctx_len, step.seq_of_token, T,
                step.num_seqs, nh, nkv, hd, self.scale, self.window if self.window else 0, plan[2], scratch,
                self._table, self.position.rotary_dim, self.position.rows_of(step), qw, kw, self.norm_eps,
                writes_cache, step.status)
            return self._project_out(o, T, defer)
        if self._table is not None or type(self.position).apply is PositionEncoding.apply:
            # one kernel: norm, rotation by the table's rows, cache write
            native.qknorm_rope_kvwrite(
                qkv, nh, nkv, hd, qw, kw, self.norm_eps, self._table,
                self.position.rotary_dim if self._table is not None else 0,
                self.position.rows_of(step), step.seq_of_token, bt, cache.page_size, kp, vp, step.status)
        else:
            # a position encoding of its own making: norm, then the part's ``apply``, then the write
            if self.qk_norm:
                native.qk_headnorm(qkv, nh, nkv, hd, qw, kw, self.norm_eps, step.seq_of_token)
            self.position.apply(qkv[:, :nh * hd].view(T, nh, hd), qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd), step)
            if kp is not None:
                native.qknorm_rope_kvwrite(qkv, nh, nkv, hd, None, None, 0.0, None, 0, step.positions,
                                           step.seq_of_token, bt, cache.page_size, kp, vp, step.status)
        self.attend(o, qkv, step, cache, bt)
        return self._project_out(o, T, defer)

    def _project_out(self, o, T, defer):
        out = self.rt.workspace.get("attn.out", (T, self.hidden_size), self.rt.dtype)
        if defer and may_defer(o, self.w_o_weight):
            return PendingProduct(o, self.w_o_weight, None, out)
        return linear(o, self.w_o_weight, None, out)

    def _rotates_in_decode(self, step, cache) -> bool:
        """Every request of the step brings one token, the position encoding is a table of angles, and
        the decode attention kernel takes these sizes with norm, rotation and cache write inside."""
        if step.max_q_len != 1 or step.num_tokens != step.num_seqs or self._table is None or step.plan_for_any_batch:
            return False
        if self.rt.dtype != torch.bfloat16 or not native.flash_supports(self.hd, self.rt.dtype):
            return False
        return native.flash_rotating_supports(self.hd, cache.page_size, cache.k_pages.shape[0], self.nh, self.nkv,
                                              self.position.rotary_dim)

    def launch_plan(self, step):
        """The attention kernels' plan for this step: tile counts and the number of splits along the
        keys, from the step's shape and its longest context.  Layers of equal sizes share it."""
        if not native.flash_supports(self.hd, self.rt.dtype):
            return None
        if self._long_rows is None:
            self._long_rows = native.LONG_ROWS if (not self.window and native.flash_has_tc(self.hd)) else 0
        long_rows = self._long_rows
        key = ("flash", self.nh, self.nkv, long_rows)
        plan = step.plans.get(key)
        if plan is None:
            if step.plan_for_any_batch:
                plan = native.flash_plan_for_any(step.num_tokens, step.num_seqs, self.nh // self.nkv, self.nkv,
                                                 step.max_ctx_len, long_rows=long_rows)
            else:
                plan = native.flash_plan(step.q_lens, self.nh // self.nkv, self.nkv, step.max_ctx_len,
                                         long_rows=long_rows)
            step.plans[key] = plan
        return plan

    def attend(self, o, qkv, step, cache, bt) -> None:
        """Chooses the attention kernel for this step's tokens: the tensor-core kernel for
        bfloat16 and head sizes in steps of 16, else the 32-bit kernel that takes any size."""
        if native.flash_supports(self.hd, qkv.dtype):
            T = o.shape[0]
            plan = self.launch_plan(step)
            scratch = None
            if plan[2] > 1:
                n = native.flash_scratch_elems(T, self.nh, self.hd, plan[2])
                scratch = self.rt.workspace.get("attn.splits", (n,), torch.float32)
            native.flash_attention(
                o, qkv, qkv.shape[1], cache.k_pages, cache.v_pages, bt, step.cu_q, step.ctx_len,
                step.seq_of_token, T, step.num_seqs, self.nh, self.nkv, self.hd, self.scale,
                self.window if self.window else 0, plan, scratch)
            return
        native.paged_attention_generic(
            o, qkv, qkv.shape[1], cache.k_pages, cache.v_pages, bt, step.positions,
            step.seq_of_token, o.shape[0], self.nh, self.nkv, self.hd, self.scale,
            self.window if self.window else 0)
