"""Mixers: the part of a layer that lets tokens see other tokens.

Interface of the family:

* ``cache_spec()`` — ``KVSpec``, ``StateSpec`` or None: what one layer of this
  mixer keeps per sequence.  The cache groups layers with equal needs.
* ``forward(x, step, cache) -> y`` — ``x`` [T, hidden] in the compute dtype
  (``y`` may be a stack of 32-bit partial sums [S, T, hidden]: see ``Norm.add_norm``),
  ``step`` the ``StepContext`` (which sequence and position each row has),
  ``cache`` the layer's view of its store (``KVLayerView`` / ``StateLayerView``).
  It must store what later steps need (keys, values, state) for the rows of
  sequences whose slot is not negative, and return [T, hidden].
  A mixer with a recurrence walks each sequence's rows in order, using
  ``step.cu_q``; it must give the same state whether the tokens come in one
  step or one by one.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..cache.spec import KVSpec
from ..kernels import ops
from .base import BuildContext, ParamSpec, Part, PartSpec, build_part, register_part
from .linear import Linear
from .position import PositionEncoding


class Mixer(Part):
    family = "mixer"

    def cache_spec(self):
        return None

    def forward(self, x, step, cache):
        raise NotImplementedError


@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    """Causal grouped-query attention over the paged cache.

    q, k, v projections without bias (fused into one product at load, as the
    reference fuses them, src/model.rs:1396, 6021-6073); optional RMSNorm of
    every q and k head over head_dim with one weight vector shared by the heads,
    before the rotation (src/training.rs:318-331); the position encoding of the
    given spec; k and v stored at the token's position; scores q.k * scale with
    scale = 1/sqrt(head_dim) unless given (src/model.rs:2398); query head h reads
    kv head h // (heads / kv_heads) (src/kernels.rs:1166); keys up to the query's
    own position, or the last ``window`` of them; o projection.
    """

    def __init__(self, ctx: BuildContext, hidden: int, n_heads: int, n_kv_heads: int,
                 head_dim: int, position: PartSpec, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, scale: Optional[float] = None,
                 shares_kv: bool = False):
        super().__init__(ctx)
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} kv heads")
        self.hidden, self.nq, self.nkv, self.D = int(hidden), int(n_heads), int(n_kv_heads), int(head_dim)
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.D)
        # a layer that attends over another layer's keys and values projects
        # queries only, stores nothing and owns no cache (the schedule says whose
        # cache it is given)
        self.shares_kv = bool(shares_kv)
        self.position = build_part("position", position, ctx)
        self.qkv = self.o = None
        self.q_norm_w = self.k_norm_w = None

    def children(self):
        return (self.position,)

    def param_specs(self):
        H, nq, nkv, D = self.hidden, self.nq, self.nkv, self.D
        specs = {"q_proj.weight": ParamSpec((nq * D, H)), "o_proj.weight": ParamSpec((H, nq * D))}
        if not self.shares_kv:
            specs["k_proj.weight"] = ParamSpec((nkv * D, H))
            specs["v_proj.weight"] = ParamSpec((nkv * D, H))
        if self.qk_norm_eps is not None:
            specs["q_norm.weight"] = ParamSpec((D,), "vector")
            if not self.shares_kv:
                specs["k_norm.weight"] = ParamSpec((D,), "vector")
        return specs

    def load(self, params):
        ws = [params["q_proj.weight"]]
        if not self.shares_kv:
            ws += [params["k_proj.weight"], params["v_proj.weight"]]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("q, k and v projections must be stored in one dtype to be fused")
        self.qkv = Linear(torch.cat(ws, dim=0) if len(ws) > 1 else ws[0], self.ctx.products)
        self.o = Linear(params["o_proj.weight"], self.ctx.products)
        if self.qk_norm_eps is not None:
            self.q_norm_w = params["q_norm.weight"].contiguous()
            if not self.shares_kv:
                self.k_norm_w = params["k_norm.weight"].contiguous()

    def kernel_modules(self):
        mods = ("qk_prepare", "attn_generic") + self.qkv.kernel_modules() + self.o.kernel_modules()
        if self.ctx.dtype == torch.bfloat16:
            mods += ops.fast_attention_modules(self.D, self.nq, self.nkv)
        return mods

    def cache_spec(self):
        return None if self.shares_kv else KVSpec(self.nkv, self.D, self.window)

    def captures_prompts(self):
        # an encoding with arithmetic of its own runs between two kernels here and
        # answers for itself
        return True

    def forward(self, x, step, cache):
        T = x.shape[0]
        rot = self.position.rotary()
        if cache is None or (cache.spec.n_kv_heads, cache.spec.head_dim) != (self.nkv, self.D):
            raise ValueError(f"attention with {self.nkv} kv heads of {self.D} was given the cache "
                             f"{None if cache is None else cache.spec}")
        fused = rot is not None or type(self.position).apply_qk is PositionEncoding.apply_qk
        # the q/k preparation can add the partial sums of a split-K projection itself
        qkv = self.qkv(x, partial_ok=fused and x.dtype == torch.bfloat16 and not self.shares_kv)
        if self.shares_kv:
            q, _ = ops.qk_prepare(qkv, self.nq, 0, self.D, q_w=self.q_norm_w,
                                  eps=self.qk_norm_eps or 0.0,
                                  inv_freq=rot.inv_freq if rot else None,
                                  rot_dim=rot.rot_dim if rot else 0, token_seq=step.token_seq,
                                  token_pos=step.token_pos, slots=step.slots)
            if rot is None:
                q, _k = self.position.apply_qk(q, q[:, :0], step.token_pos)
            attn = ops.attention(q.contiguous(), cache.k_pages, cache.v_pages, cache.block_table,
                                 step=step, page=cache.page, scale=self.scale, window=self.window)
            return self.o(attn.view(T, self.nq * self.D), partial_ok=True)
        common = dict(q_w=self.q_norm_w, k_w=self.k_norm_w, eps=self.qk_norm_eps or 0.0,
                      token_seq=step.token_seq, token_pos=step.token_pos, slots=step.slots)
        if fused:
            q, _ = ops.qk_prepare(qkv, self.nq, self.nkv, self.D,
                                  inv_freq=rot.inv_freq if rot else None,
                                  rot_dim=rot.rot_dim if rot else 0,
                                  block_table=cache.block_table, k_pages=cache.k_pages,
                                  v_pages=cache.v_pages, page=cache.page, **common)
        else:
            # a position encoding with its own arithmetic: normalise, hand q and k
            # over, then store
            q, kv = ops.qk_prepare(qkv, self.nq, self.nkv, self.D, want_kv_out=True, **common)
            k, v = kv[:, :self.nkv], kv[:, self.nkv:]
            q, k = self.position.apply_qk(q, k, step.token_pos)
            kv = torch.cat([k, v], dim=1).contiguous()
            ops.kv_write(kv, self.nkv, self.D, token_seq=step.token_seq, token_pos=step.token_pos,
                         slots=step.slots, block_table=cache.block_table, k_pages=cache.k_pages,
                         v_pages=cache.v_pages, page=cache.page)
            q = q.contiguous()
        attn = ops.attention(q, cache.k_pages, cache.v_pages, cache.block_table, step=step,
                             page=cache.page, scale=self.scale, window=self.window)
        return self.o(attn.view(T, self.nq * self.D), partial_ok=True)
