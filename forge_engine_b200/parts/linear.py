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

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, status=None) -> None:
        """``status`` is the device status word; without it the tcgen05 kernel is not used."""
        self.status = status
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.bias = None if bias is None else bias.float().contiguous()
        self._bias_model = None if bias is None else bias.to(weight.dtype).contiguous()

    def _tc5_ok(self, x: torch.Tensor) -> bool:
        return (x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16
                and x.shape[0] <= native.TC5_MAX_ROWS and self.in_features % 8 == 0 and self.status is not None)

    def __call__(self, x: torch.Tensor, out_dtype=None) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        n = x.shape[0]
        if self._tc5_ok(x) and out_dtype in (torch.bfloat16, torch.float32):
            out = torch.empty((n, self.out_features), dtype=out_dtype, device=x.device)
            mode = native.TC5_STORE_BF16 if out_dtype == torch.bfloat16 else native.TC5_STORE_F32
            native.gemm_tc5(x, self.weight, out, mode, self.status, bias=self.bias,
                            ksplit=native.tc5_ksplit(self.out_features, self.in_features))
            return out
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


    def silu_mul(self, x: torch.Tensor, interleave: int) -> torch.Tensor | None:
        """For a weight whose rows alternate ``interleave`` gate and up features: returns
        silu(gate) * up [n, out/2] from the fused tcgen05 epilogue, or None if that kernel
        does not take this call (then the caller multiplies after a plain product)."""
        if interleave != 16 or not self._tc5_ok(x) or self.out_features % 32 or self.bias is not None:
            return None
        out = torch.empty((x.shape[0], self.out_features // 2), dtype=torch.bfloat16, device=x.device)
        native.gemm_tc5(x, self.weight, out, native.TC5_SILU_MUL, self.status,
                        ksplit=native.tc5_ksplit(self.out_features, self.in_features))
        return out


def interleave_rows(gate: torch.Tensor, up: torch.Tensor, block: int) -> torch.Tensor:
    """Rows [block of gate, block of up, block of gate, ...]; both are [I, H] with I % block == 0."""
    if gate.dtype != up.dtype:
        gate, up = gate.float(), up.float()
    inter, hidden = gate.shape
    stacked = torch.stack((gate.view(inter // block, block, hidden), up.view(inter // block, block, hidden)), dim=1)
    return stacked.reshape(2 * inter, hidden).contiguous()


def fuse_rows(tensors: list) -> torch.Tensor:
    """Concatenate ``[out_i, in]`` matrices (or bias vectors) along rows; if their dtypes
    differ, all are raised to 32-bit first (exact for bfloat16)."""
    dtypes = {t.dtype for t in tensors}
    if len(dtypes) > 1:
        tensors = [t.float() for t in tensors]
    return torch.cat(tensors, dim=0).contiguous()
