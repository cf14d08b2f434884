"""Differentiable SpMM: C = A · B with gradients for B and for the stored values of A.

The reference stops at the forward operator (spmm_forward_fp16_tcu_cuda_sptc_mma_parallel_online,
TR-source/SpMM/mGCN_online.cpp:760); it has no backward pass and no transpose.  For training
the two adjoints are
    dB       = Aᵀ · dC                      -> the same fused SpMM over the format of Aᵀ
    dval[e]  = < dC[row(e), :], B[col(e), :] >  -> planned SDDMM on A's pattern (trs_sddmm_plan_run)
Both formats are built lossless (strict mode): the reference-compatible format drops the third and
fourth non-zero of a row inside a 4-column group, and the dropped sets of A and Aᵀ differ, so the
lossy pair would not be adjoint to each other.
"""
from __future__ import annotations

import torch

from .builder import build_format
from .sddmm import SddmmPlan
from .spmm import SpmmPlan


def transpose_csr(rowptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor | None, n_cols: int):
    """CSR of the transpose (canonical: columns ascending inside a row), on the inputs' device.
    Returns (rowptr_t, col_t, val_t, perm) with perm[e_t] = entry of A that became entry e_t."""
    n_rows = rowptr.numel() - 1
    deg = (rowptr[1:] - rowptr[:-1]).long()
    rows = torch.repeat_interleave(torch.arange(n_rows, device=rowptr.device), deg)
    perm = torch.sort(col.long(), stable=True).indices      # stable: rows stay ascending per column
    rp_t = torch.zeros(n_cols + 1, dtype=torch.long, device=rowptr.device)
    rp_t[1:] = torch.cumsum(torch.bincount(col.long(), minlength=n_cols), 0)
    return rp_t.to(rowptr.dtype), rows[perm].to(col.dtype), (val[perm] if val is not None else None), perm


class _SpmmFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, op, values, B):
        ctx.op = op
        ctx.save_for_backward(B)
        ctx.values_need_grad = values is not None and values.requires_grad
        return op.plan.run(B.contiguous(), out_dtype=torch.float16)

    @staticmethod
    def backward(ctx, dC):
        op = ctx.op
        (B,) = ctx.saved_tensors
        dC = dC.contiguous().half()
        dB = op.plan_t.run(dC, out_dtype=torch.float16) if ctx.needs_input_grad[2] else None
        dval = None
        if ctx.values_need_grad:
            dval = op.sddmm_plan().run(dC, B.contiguous()).float()
        return None, dval, dB


class DifferentiableSpmm:
    """A fixed sparsity pattern with its forward and transposed formats resident on the GPU.

    op = DifferentiableSpmm(rowptr, col, val, n_cols); C = op(B) is fp16 [n_rows, F] and
    back-propagates into B.  Pass `values=` (a leaf tensor equal to `val`) to op(...) to also get
    the gradient with respect to the stored values; the numbers used in the forward pass are the
    ones the format was built from."""

    def __init__(self, rowptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor, n_cols: int, **build_kwargs):
        if rowptr.device.type != "cuda":
            raise ValueError("DifferentiableSpmm needs CUDA tensors (there is no CPU fallback)")
        self.rowptr, self.col = rowptr.contiguous(), col.contiguous()
        self.n_rows, self.n_cols = rowptr.numel() - 1, int(n_cols)
        build_kwargs["strict"] = True
        self.format, self.stats = build_format(self.rowptr, self.col, val.float().contiguous(), **build_kwargs)
        self.plan = SpmmPlan(self.format, self.n_rows, self.n_cols)
        rp_t, col_t, val_t, _ = transpose_csr(self.rowptr, self.col, val.float(), self.n_cols)
        self.format_t, self.stats_t = build_format(rp_t.contiguous(), col_t.contiguous(), val_t.contiguous(),
                                                   **build_kwargs)
        self.plan_t = SpmmPlan(self.format_t, self.n_cols, self.n_rows)
        self._sddmm_plan = None

    def sddmm_plan(self) -> SddmmPlan:
        """Planned SDDMM over A's pattern (built on first use: only callers that ask for the gradient
        of the stored values need it)."""
        if self._sddmm_plan is None:
            self._sddmm_plan = SddmmPlan(self.rowptr, self.col, self.n_cols)
        return self._sddmm_plan

    def __call__(self, B: torch.Tensor, values: torch.Tensor | None = None) -> torch.Tensor:
        if B.dtype != torch.float16 or B.dim() != 2 or B.shape[0] != self.n_cols:
            raise ValueError("B must be fp16 [n_cols, F]")
        return _SpmmFn.apply(self, values, B)
