"""y = x W^T with W stored [out, in], the one linear layer every part uses.

It picks the product by the weight's precision and by the number of rows:

* 32-bit weight: the true 32-bit CUDA-core product (``gemm_f32``); bf16
  activations are widened first and the result narrowed, so a tensor that the
  checkpoint stores in 32-bit is used in 32-bit.
* bf16 weight, up to 64 rows (every decode step): the TMA-fed tcgen05 product
  with the weight rows on the 128-row side of the MMA (``gemm_tc_bf16`` with
  ``swap``), or, for ``products.decode = "skinny"``, the mma.sync weight-streaming
  kernel (``gemm_skinny_bf16``).
* bf16 weight, more rows (a prompt): ``products.prefill = "auto"`` takes the product
  on pairs of SMs (``gemm_tc2_bf16``, tcgen05.mma.cta_group::2) where it is at
  least as fast as the library's product, which is the fused gate|up product with
  its SiLU epilogue when its rounds of 256 x 256 tiles on the GPU's pairs of SMs
  are mostly full (``ops.gemm_tc2_pays`` has the measurements), and the library's
  product elsewhere, where the reference uses a library too (cuBLAS GemmEx,
  src/cublas.rs:287-307).  ``"pair"`` takes the pair product for everything it can
  store, ``"tc"`` the single-SM tcgen05 kernel in its other orientation,
  ``"library"`` the library throughout.  Measured at 2,048 rows (us, library /
  pair): qkv 46 / 47, o 35 / 48, gate|up 140 + 24 for SiLU / 149 fused, down 73 / 102
  (o and down are 80 tiles on 74 pairs of SMs: a second round for six tiles).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import ProductChoice


class Linear:
    def __init__(self, weight: torch.Tensor, products: Optional[ProductChoice] = None):
        """``products``: which kernels take the products (a part passes
        ``ctx.products``); None means the defaults."""
        products = products or ProductChoice()
        self.decode_kernel, self.prefill_kernel = products.decode, products.prefill
        if weight.dim() != 2:
            raise ValueError(f"a linear weight is [out, in], got {tuple(weight.shape)}")
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"a linear weight is float32 or bfloat16, got {weight.dtype}")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape

    def kernel_modules(self):
        if self.weight.dtype == torch.float32:
            return ("gemm_f32", "elementwise")
        if self.in_features % 8:
            return ()                                  # only the library's product takes such a width
        mods = ("gemm_tc",) if "tc" in (self.decode_kernel, self.prefill_kernel) else ()
        if self.decode_kernel == "skinny":
            mods += ("gemm_skinny_bf16",)
        if self.prefill_kernel in ("auto", "pair"):
            mods += ("gemm_tc2",)
        return mods

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                 partial_ok: bool = False) -> torch.Tensor:
        """``partial_ok``: the caller hands the result to a kernel that can add
        32-bit partial sums (a norm's residual add, the q/k preparation); a product
        with few rows and few tiles may then come back as [S, M, N] float32, its
        split-K reduction left to that kernel."""
        out_dtype = out_dtype or x.dtype
        w = self.weight
        if w.dtype == torch.float32:
            y = ops.gemm_f32(ops.cast(x, torch.float32), w)
            return ops.cast(y, out_dtype)
        if x.dtype != torch.bfloat16:
            raise ops.KernelError("a bfloat16 weight takes bfloat16 activations")
        M = x.shape[0]
        if self.in_features % 8 == 0:
            if M <= ops.SKINNY_MAX_ROWS:
                if self.decode_kernel == "tc":
                    return ops.gemm_tc_bf16(x, w, out_dtype, swap=True, split_out=partial_ok)
                return ops.gemm_skinny_bf16(x, w, out_dtype)
            if self.prefill_kernel == "tc":
                return ops.gemm_tc_bf16(x, w, out_dtype, swap=False)
            if ops.gemm_tc2_takes(self.out_features, out_dtype) and (
                    self.prefill_kernel == "pair" or
                    (self.prefill_kernel == "auto" and
                     ops.gemm_tc2_pays(M, self.out_features, x.device, fused_silu=False))):
                return ops.gemm_tc2_bf16(x, w, out_dtype)
        return ops.library_mm(x, w, out_dtype)

    def silu_mul(self, x: torch.Tensor, interleave: int) -> torch.Tensor:
        """silu(gate) * up of a fused gate|up weight.  ``interleave`` 0: gate rows
        first, then up rows; 8: groups of 8 gate rows followed by their 8 up rows,
        which lets the decode kernel finish the product in its epilogue."""
        w = self.weight
        if (interleave == 8 and w.dtype == torch.bfloat16 and x.shape[0] <= ops.SKINNY_MAX_ROWS
                and self.in_features % 8 == 0):
            if self.decode_kernel == "tc":
                return ops.gemm_tc_bf16(x, w, x.dtype, swap=True, silu_mul=True)
            return ops.gemm_skinny_bf16(x, w, x.dtype, silu_mul=True)
        if (interleave == 8 and w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
                and self.in_features % 8 == 0 and self.out_features % 32 == 0
                and (self.prefill_kernel == "pair" or
                     (self.prefill_kernel == "auto" and
                      ops.gemm_tc2_pays(x.shape[0], self.out_features, x.device, fused_silu=True)))):
            return ops.gemm_tc2_bf16(x, w, x.dtype, silu_mul=True)
        return ops.silu_mul(self(x), interleave)
