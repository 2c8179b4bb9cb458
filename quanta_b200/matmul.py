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


# The library's kernels for products of fewer rows than this are slower than its kernel for this many
# (measured on B200, weights from HBM: 3072 x 6144 at 8 rows 37 us, at 32 rows 27 us), so activations of
# small steps are laid out with spare rows and multiplied as MIN_ROWS rows.  Rows do not mix in a
# product: what the spare rows hold never reaches a real row.
MIN_ROWS = 32


def empty_rows(n: int, *cols: int, dtype: torch.dtype, device) -> torch.Tensor:
    """``[n, *cols]`` uninitialised, as the first rows of a buffer of at least MIN_ROWS rows, which
    ``linear`` finds again by the size of the storage."""
    return torch.empty((max(n, MIN_ROWS), *cols), dtype=dtype, device=device)[:n]


def _with_spare_rows(x: torch.Tensor) -> torch.Tensor:
    n, k = x.shape
    if (0 < n < MIN_ROWS and x.is_cuda and x.is_contiguous() and x.storage_offset() == 0
            and x.untyped_storage().nbytes() >= MIN_ROWS * k * x.element_size()):
        return torch.as_strided(x, (MIN_ROWS, k), (k, 1))
    return x


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x [T, in] @ w [out, in].T``; accumulation is float32; ``out_dtype`` float32 keeps the
    accumulator's precision for bfloat16 operands.  An ``x`` from ``empty_rows`` is multiplied with its
    spare rows and the result cut back to ``T`` rows."""
    n = x.shape[0]
    xp = _with_spare_rows(x)
    if xp is not x:
        return linear(xp, w, out_dtype)[:n]
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, w.t(), out_dtype=out_dtype)
    return torch.mm(x, w.t())
