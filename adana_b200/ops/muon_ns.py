"""Newton–Schulz orthogonalisation (Muon's inner loop) as a chain of tcgen05 GEMMs.

One quintic iteration X <- aX + (bA + cA²)X with A = XXᵀ (reference src/optim/muon.py:19-47) is three
tensor-core GEMMs whose scale-and-add terms live in the GEMM epilogue, so an iteration makes exactly three
kernel launches and no elementwise passes:

    A  = X · Xᵀ                         (plain bf16 epilogue; X is read K-major for both operands)
    B  = c · (A · Aᵀ) + b · A           (A is symmetric, so A·Aᵀ = A²; `EPI_AXPBY_BF16` adds b·A)
    X' = 1 · (B · X) + a · X            (X read as the MN-major right operand; `EPI_AXPBY_BF16` adds a·X)

X ping-pongs between two buffers because every output tile of the third GEMM reads all of X.
`newton_schulz5` in `adana_b200/optim/muon.py` is the PyTorch oracle the GPU test compares against.
"""
from __future__ import annotations

import torch

from . import _lib
from .gemm import EPI_AXPBY_BF16, EPI_BF16, gemm

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def supported(G: torch.Tensor) -> bool:
    """2-D CUDA matrices whose two extents are multiples of 8 (16-byte rows for the TMA descriptors)."""
    return (G.is_cuda and G.dim() == 2 and G.size(0) % 8 == 0 and G.size(1) % 8 == 0 and _lib.available()
            and G.dtype in (torch.bfloat16, torch.float32, torch.float16))


def newton_schulz5_cuda(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    a, b, c = NS_COEFFS
    tall = G.size(0) > G.size(1)
    X = (G.T if tall else G).to(torch.bfloat16)
    X = (X / (X.norm() + eps)).contiguous()
    m, n = X.shape
    Y = torch.empty_like(X)
    A = torch.empty((m, m), dtype=torch.bfloat16, device=X.device)
    B = torch.empty_like(A)
    for _ in range(steps):
        gemm(X, X, A, M=m, N=m, K=n, epi=EPI_BF16)
        gemm(A, A, B, M=m, N=m, K=m, epi=EPI_AXPBY_BF16, R=A, alpha=c, beta=b)
        gemm(B, X, Y, M=m, N=n, K=m, b_mn=True, epi=EPI_AXPBY_BF16, R=X, alpha=1.0, beta=a)
        X, Y = Y, X
    return X.T if tall else X
