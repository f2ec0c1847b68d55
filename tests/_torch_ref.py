"""Test-only torch restatement of the reference Newton-Schulz arithmetic, used on the GPU at sizes where the
numpy oracle would take minutes.  It follows emerging_optimizers/orthogonalized_optimizers/muon_utils.py:205-274,
348-378 of the reference: normalise, optional bf16 cast, then matmul / addmm per step with library GEMMs."""

import torch

from oracle import ns_oracle


def newton_schulz_torch(x, steps, coefficient_type="quintic", bf16=True, eps=1e-15):
    transpose = x.size(-2) > x.size(-1)
    if transpose:
        x = x.mT
    X = torch.nn.functional.normalize(x, p=2, dim=(-2, -1), eps=eps)
    if bf16:
        X = X.to(torch.bfloat16)
    for a, b, c in ns_oracle.coefficient_schedule(steps, coefficient_type):
        A = X @ X.mT
        if c != 0.0:
            B = torch.baddbmm(A, A, A, alpha=c, beta=b) if X.ndim == 3 else torch.addmm(A, A, A, alpha=c, beta=b)
            X = torch.baddbmm(X, B, X, alpha=1.0, beta=a) if X.ndim == 3 else torch.addmm(X, B, X, alpha=1.0, beta=a)
        else:
            X = torch.baddbmm(X, A, X, alpha=b, beta=a) if X.ndim == 3 else torch.addmm(X, A, X, alpha=b, beta=a)
    X = X.to(torch.float32)
    return X.mT if transpose else X


def rel_fro(a, b):
    a = a.double()
    b = b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def int_tensor(*shape, seed=0, lo=-3, hi=4, dtype=torch.bfloat16, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(lo, hi, shape, generator=g).to(dtype).to(device)


def randn_tensor(*shape, seed=0, scale=1.0, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(device)
