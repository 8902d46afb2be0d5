"""Shared helpers for the parity tests: seeded synthetic inputs with the value distributions of
the benchmark configurations, and the tolerance check."""
from __future__ import annotations

import torch

from oracle import gdn as ogdn
from oracle import tables as otab


def synth_gdn_inputs(B, T, H, K, V, seed=0, dtype=torch.bfloat16, normalize_qk=True):
    """q,k,v ~ N(0,1) (q,k L2-normalised per head), beta = sigmoid(N(0,1)), g = -softplus(N(0,1)),
    generated in fp32 on CPU and cast."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=gen)
    k = torch.randn(B, T, H, K, generator=gen)
    v = torch.randn(B, T, H, V, generator=gen)
    if normalize_qk:
        q, k = ogdn.l2norm(q), ogdn.l2norm(k)
    beta = torch.randn(B, T, H, generator=gen).sigmoid()
    g = -torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen))
    h0 = torch.randn(B, H, K, V, generator=gen) * 0.1
    return q.to(dtype), k.to(dtype), v.to(dtype), g, beta.to(dtype), h0


def synth_mamba_inputs(B, T, H, K, V, seed=0, dtype=torch.bfloat16):
    """x ~ N(0,1); dt = softplus(N(-2,1)); A = -exp(U(0, ln 16)); v = x*dt, g = A*dt;
    B, C ~ N(0, 1/sqrt(K)) per head."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, H, V, generator=gen)
    dt = torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen) - 2.0)
    A = -torch.exp(torch.rand(H, generator=gen) * torch.log(torch.tensor(16.0)))
    k = torch.randn(B, T, H, K, generator=gen) * K ** -0.25
    q = torch.randn(B, T, H, K, generator=gen) * K ** -0.25
    v = x * dt[..., None]
    g = A.view(1, 1, H) * dt
    h0 = torch.randn(B, H, K, V, generator=gen) * 0.1
    return q.to(dtype), k.to(dtype), v.to(dtype), g, h0


def assert_close(got: torch.Tensor, ref: torch.Tensor, tol: float, what: str = ""):
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs()
    bound = tol + tol * ref.abs()
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())}/{bad.numel()} elements outside rtol=atol={tol}; "
                           f"max abs err {err.max().item():.4g} (ref max {ref.abs().max().item():.4g})")
