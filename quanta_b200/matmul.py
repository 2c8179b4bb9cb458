"""Dense projections through the library GEMM (cuBLAS via torch), as the reference does its own
(``nn.Linear``, src/quanta/minimax/attention.py:166-169).

float32 products run as true float32: TF32 and reduced-precision accumulation are switched off
process-wide when the first engine is built.
"""

from __future__ import annotations

import torch

_configured = False


def configure() -> None:
    global _configured
    if _configured:
        return
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    _configured = True


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x [T, in] @ w [out, in].T``; accumulation is float32; ``out_dtype`` float32 keeps the
    accumulator's precision for bfloat16 operands."""
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, w.t(), out_dtype=out_dtype)
    return torch.mm(x, w.t())
