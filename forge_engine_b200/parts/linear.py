"""y = x W^T (+ b) for an ``[out, in]`` weight kept in the dtype it was stored in.

Which kernel runs is decided by the dtypes alone:

* weight and input both bfloat16 - the tensor-core product (library GEMM, as upstream
  uses ``nn.Linear`` for every projection, src/forge_engine/qwen3.py:113-122);
* anything else (the 32-bit path, or a tensor the checkpoint stores in 32-bit) - the
  plain FFMA kernel, which never uses a reduced-precision matrix mode.
"""

from __future__ import annotations

import os

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


    def adds_into(self, x: torch.Tensor, residual: torch.Tensor) -> bool:
        """Whether ``add_into`` works for an input with ``x``'s dtype and row count."""
        return (self._tc5_ok(x) and residual.dtype == torch.float32 and residual.is_contiguous()
                and os.environ.get("FORGE_ENGINE_ADD_EPILOGUE", "1") != "0")

    def add_into(self, x: torch.Tensor, residual: torch.Tensor) -> bool:
        """residual (32-bit [n, out]) += x W^T in the product's own epilogue, if the tcgen05
        kernel takes the call (then True); otherwise nothing happens."""
        if not self.adds_into(x, residual):
            return False
        native.gemm_tc5(x, self.weight, residual, native.TC5_ADD_F32, self.status, bias=self.bias,
                        ksplit=native.tc5_ksplit_add(self.out_features, self.in_features))
        return True

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


def fused_rows(weights, names: list, rows: list) -> torch.Tensor:
    """``weights[name]`` for the names in order, stacked along rows (``rows[i]`` of them
    each) into one tensor that is allocated first.  Each source is looked up when its turn
    comes and dropped once copied: with a mapping that reads tensors on access, only one
    source exists beside the result at any time.  Sources stored in different dtypes make
    the result 32-bit (exact for bfloat16)."""
    out, at = None, 0
    for name, count in zip(names, rows):
        tensor = weights[name]
        if tensor.shape[0] != count:
            raise ValueError(f"{name}: {tensor.shape[0]} rows, {count} expected")
        if out is None:
            out = torch.empty((sum(rows), *tensor.shape[1:]), dtype=tensor.dtype, device=tensor.device)
        elif tensor.dtype != out.dtype and out.dtype != torch.float32:
            out = out.float()
        out[at : at + count].copy_(tensor)
        at += count
        del tensor
    return out


def interleaved_rows(weights, gate_name: str, up_name: str, inter: int, block: int) -> torch.Tensor:
    """``interleave_rows`` of two ``[inter, hidden]`` tensors looked up one after the other
    and copied straight into the result."""
    out = None
    for index, name in enumerate((gate_name, up_name)):
        tensor = weights[name]
        if out is None:
            out = torch.empty((2 * inter, tensor.shape[1]), dtype=tensor.dtype, device=tensor.device)
        elif tensor.dtype != out.dtype and out.dtype != torch.float32:
            out = out.float()
        out.view(inter // block, 2, block, tensor.shape[1])[:, index].copy_(tensor.view(inter // block, block, -1))
        del tensor
    return out


def interleave_rows(gate: torch.Tensor, up: torch.Tensor, block: int) -> torch.Tensor:
    """Rows [block of gate, block of up, block of gate, ...]; both are [I, H] with I % block == 0."""
    if gate.dtype != up.dtype:
        gate, up = gate.float(), up.float()
    inter, hidden = gate.shape
    stacked = torch.stack((gate.view(inter // block, block, hidden), up.view(inter // block, block, hidden)), dim=1)
    return stacked.reshape(2 * inter, hidden).contiguous()
