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


def ns_chain(X: torch.Tensor, Y: torch.Tensor, A: torch.Tensor, B: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """`steps` quintic iterations on X [m, n] (bf16, contiguous, Frobenius norm <= 1) without any transpose in memory.
    Y has X's shape, A and B are [s, s] with s = min(m, n).  A wide matrix (m <= n) iterates X <- (bA + cA^2) X + aX
    with A = X X^T; a tall one uses the Gram matrix of the other side, A = X^T X (read MN-major by the GEMM) and
    X <- X (bA + cA^2) + aX, which is the same map applied to X^T.  Returns whichever of X / Y holds the result."""
    a, b, c = NS_COEFFS
    m, n = X.shape
    for _ in range(steps):
        if m <= n:
            gemm(X, X, A, M=m, N=m, K=n, epi=EPI_BF16)
            gemm(A, A, B, M=m, N=m, K=m, epi=EPI_AXPBY_BF16, R=A, alpha=c, beta=b)
            gemm(B, X, Y, M=m, N=n, K=m, b_mn=True, epi=EPI_AXPBY_BF16, R=X, alpha=1.0, beta=a)
        else:
            gemm(X, X, A, M=n, N=n, K=m, a_mn=True, b_mn=True, epi=EPI_BF16)
            gemm(A, A, B, M=n, N=n, K=n, epi=EPI_AXPBY_BF16, R=A, alpha=c, beta=b)
            gemm(X, B, Y, M=m, N=n, K=n, epi=EPI_AXPBY_BF16, R=X, alpha=1.0, beta=a)
        X, Y = Y, X
    return X


def newton_schulz5_cuda(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    X = G.to(torch.bfloat16)
    X = (X / (X.norm() + eps)).contiguous()
    s = min(X.shape)
    A = torch.empty((s, s), dtype=torch.bfloat16, device=X.device)
    return ns_chain(X, torch.empty_like(X), A, torch.empty_like(A), steps)
