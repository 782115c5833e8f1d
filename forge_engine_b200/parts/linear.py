"""y = x W^T (+ b) for an ``[out, in]`` weight kept in the dtype it was stored in.

Which kernel runs is decided by the dtypes alone:

* weight and input both bfloat16 - the tensor-core product (library GEMM, as upstream
  uses ``nn.Linear`` for every projection, src/forge_engine/qwen3.py:113-122);
* anything else (the 32-bit path, or a tensor the checkpoint stores in 32-bit) - the
  plain FFMA kernel, which never uses a reduced-precision matrix mode.
"""

from __future__ import annotations

import torch

from ..ops import native

_MM_HAS_OUT_DTYPE: bool | None = None


def _mm_out_dtype_works(device) -> bool:
    global _MM_HAS_OUT_DTYPE
    if _MM_HAS_OUT_DTYPE is None:
        try:
            a = torch.zeros((8, 16), dtype=torch.bfloat16, device=device)
            r = torch.mm(a, a.t(), out_dtype=torch.float32)
            _MM_HAS_OUT_DTYPE = r.dtype == torch.float32
        except Exception:
            _MM_HAS_OUT_DTYPE = False
    return _MM_HAS_OUT_DTYPE


class Linear:
    """One projection.  ``weight`` is [out, in]; ``bias`` (optional) is kept in 32-bit."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None) -> None:
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.bias = None if bias is None else bias.float().contiguous()
        self._bias_model = None if bias is None else bias.to(weight.dtype).contiguous()

    def __call__(self, x: torch.Tensor, out_dtype=None) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        n = x.shape[0]
        if x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            if out_dtype == torch.bfloat16:
                if self._bias_model is None:
                    return torch.mm(x, self.weight.t())
                return torch.addmm(self._bias_model, x, self.weight.t())
            if self.bias is None and _mm_out_dtype_works(x.device):
                return torch.mm(x, self.weight.t(), out_dtype=torch.float32)
        out = torch.empty((n, self.out_features), dtype=out_dtype, device=x.device)
        native.gemm_simt(x, self.weight, out, self.bias)
        return out


def fuse_rows(tensors: list) -> torch.Tensor:
    """Concatenate ``[out_i, in]`` matrices (or bias vectors) along rows; if their dtypes
    differ, all are raised to 32-bit first (exact for bfloat16)."""
    dtypes = {t.dtype for t in tensors}
    if len(dtypes) > 1:
        tensors = [t.float() for t in tensors]
    return torch.cat(tensors, dim=0).contiguous()
