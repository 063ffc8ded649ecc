"""Dense matrix products of the product path: the library's (cuBLAS through torch.mm), as
the reference engine uses a library for every dense projection
(crates/hi-cuda/src/runtime.rs:1118-1143, cublasGemmEx with float32 accumulation).

float32 products run with TF32 and reduced-precision reductions switched off, so the 32-bit
path is true 32-bit.
"""
from __future__ import annotations

import torch


def configure_matmul_precision() -> None:
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None,
           bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T`` (``+ bias`` [M], added to the float32 sums by the library's epilogue) for
    ``x`` [N, K] and ``weight`` [M, K].

    A weight kept in float32 while activations are bfloat16 (a tensor stored in 32-bit stays
    so) is multiplied in float32. ``out_dtype=torch.float32`` asks for a float32 result from
    bfloat16 operands (the logits).
    """
    if not x.is_cuda:
        raise RuntimeError("hi_b200 runs on a CUDA device only")
    if torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("TF32 matrix products are switched on; hi_b200 needs them off")
    if weight.dtype != x.dtype:
        y = torch.mm(x.to(torch.float32), weight.to(torch.float32).t())
        if bias is not None:
            y += bias.to(torch.float32)
        return y.to(out_dtype or x.dtype)
    if bias is not None:
        y = torch.addmm(bias.to(x.dtype), x, weight.t())
        return y if out_dtype in (None, x.dtype) else y.to(out_dtype)
    if out_dtype is not None and out_dtype != x.dtype:
        if x.dtype == torch.bfloat16 and out_dtype == torch.float32:
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        return torch.mm(x, weight.t()).to(out_dtype)
    return torch.mm(x, weight.t())
