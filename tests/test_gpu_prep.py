"""GPU tests (-m gpu) of the gated-delta-rule chunk preparation on its own: both kernels (tcgen05 for head dims 128/128,
mma.sync for the rest) against the defining formulas evaluated in fp64 on the CPU
(src/nats/ops/common/chunk_scaled_dot_kkt.py:105-126, src/nats/ops/utils/solve_tril.py:350-447,
src/nats/ops/gated_delta_rule/wy_fast.py:123-153, src/nats/ops/common/chunk_o.py:166,188,202-203)."""
import pytest
import torch

from tests.helpers import synth_gdn_inputs

pytestmark = pytest.mark.gpu


def _reference(q, k, v, g, beta, use_l2norm=True):
    """-> gcs, k_rstd, q_rstd, w, u, P in fp64, chunk by chunk."""
    B, T, H, K = k.shape
    q, k, v, g, beta = (x.double() for x in (q, k, v, g, beta))
    NT = -(-T // 64)
    pad = NT * 64 - T
    padt = lambda x: torch.nn.functional.pad(x, (0, 0) * (x.dim() - 2) + (0, pad))
    q, k, v, g, beta = padt(q), padt(k), padt(v), padt(g), padt(beta)
    krs = torch.rsqrt((k * k).sum(-1) + 1e-6) if use_l2norm else torch.ones_like(g)
    qrs = torch.rsqrt((q * q).sum(-1) + 1e-6) if use_l2norm else torch.ones_like(g)
    kn, qn = k * krs[..., None], q * qrs[..., None]
    c = lambda x: x.reshape(B, NT, 64, *x.shape[2:])
    gcs = c(g).cumsum(2)                                             # [B,NT,64,H]
    kc, qc, vc, bc = c(kn), c(qn), c(v), c(beta)
    dec = (gcs[:, :, :, None] - gcs[:, :, None, :]).permute(0, 1, 4, 2, 3)          # [B,NT,H,i,j]
    kk = torch.einsum("bnihd,bnjhd->bnhij", kc, kc)
    qk = torch.einsum("bnihd,bnjhd->bnhij", qc, kc)
    low = torch.tril(torch.ones(64, 64, dtype=torch.bool), -1)
    lowd = torch.tril(torch.ones(64, 64, dtype=torch.bool))
    A = torch.where(low, kk * dec.clamp(max=0).exp() * bc.permute(0, 1, 3, 2)[..., None], torch.zeros((), dtype=torch.float64))
    P = torch.where(lowd, qk * dec.clamp(max=0).exp(), torch.zeros((), dtype=torch.float64))
    rhs_u = (vc * bc[..., None]).permute(0, 1, 3, 2, 4)                              # [B,NT,H,64,V]
    rhs_w = (kc * (bc * gcs.exp())[..., None]).permute(0, 1, 3, 2, 4)
    M = torch.eye(64, dtype=torch.float64) + A
    u = torch.linalg.solve_triangular(M, rhs_u, upper=False)
    w = torch.linalg.solve_triangular(M, rhs_w, upper=False)
    back = lambda x: x.permute(0, 1, 3, 2, 4).reshape(B, NT * 64, H, x.shape[-1])[:, :T]
    return (gcs.reshape(B, NT * 64, H)[:, :T], krs[:, :T], qrs[:, :T], back(w), back(u), back(P))


def _run(name, q, k, v, g, beta, with_q, use_l2norm=True):
    from neuralattentionsearchlinear_b200 import _lib
    from neuralattentionsearchlinear_b200.nats_util import current_stream_ptr
    dev = torch.device("cuda")
    q, k, v, g, beta = (x.to(dev).contiguous() for x in (q, k, v, g, beta))
    B, T, H, K = k.shape
    V = v.shape[-1]
    bf = dict(dtype=torch.bfloat16, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    w, u = torch.zeros(B, T, H, K, **bf), torch.zeros(B, T, H, V, **bf)
    gcs, krs, qrs = torch.zeros(B, T, H, **f32), torch.zeros(B, T, H, **f32), torch.zeros(B, T, H, **f32)
    P = torch.zeros(B, T, H, 64, **bf)
    _lib.call(name, q.data_ptr() if with_q else None, k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
              _lib.DT_BF16 if beta.dtype == torch.bfloat16 else _lib.DT_F32, w.data_ptr(), u.data_ptr(), gcs.data_ptr(),
              krs.data_ptr(), qrs.data_ptr() if with_q else None, P.data_ptr() if with_q else None, B, T, H, K, V,
              int(use_l2norm), current_stream_ptr(dev))
    torch.cuda.synchronize()
    assert _lib.load().natsl_device_status() == 0
    return gcs, krs, qrs, w, u, P


def _check(got, ref, what, tol=1e-2):
    got, ref = got.double().cpu(), ref
    assert torch.isfinite(got).all(), what
    err = (got - ref).abs()
    lim = tol * float(ref.abs().max()) + tol * ref.abs()
    assert bool((err <= lim).all()), f"{what}: max err {err.max().item():.4g} at magnitude {ref.abs().max().item():.4g}"


@pytest.mark.parametrize("kernel", ["natsl_gdn_chunk_prep_tc", "natsl_gdn_chunk_prep_ex"])
@pytest.mark.parametrize("B,T,H,with_q,beta_f32,l2", [(2, 512, 4, True, False, True), (1, 700, 2, True, True, True),
                                                      (1, 64, 1, False, False, True), (2, 200, 3, True, False, False),
                                                      (1, 37, 2, True, False, True)])
def test_prep_against_the_formulas(kernel, B, T, H, with_q, beta_f32, l2):
    q, k, v, g, beta, _ = synth_gdn_inputs(B, T, H, 128, 128, seed=T + H, normalize_qk=l2 is False)
    if beta_f32:
        beta = beta.float()
    ref = _reference(q, k, v, g, beta, use_l2norm=l2)
    got = _run(kernel, q, k, v, g, beta, with_q, use_l2norm=l2)
    names = ("gcs", "k_rstd", "q_rstd", "w", "u", "P")
    for i, n in enumerate(names):
        if not with_q and n in ("q_rstd", "P"):
            continue
        _check(got[i], ref[i], f"{kernel}: {n}", 2e-5 if i < 3 else 1e-2)


def test_prep_strong_decay_and_large_beta():
    """Decays of several units per token (exponent differences of hundreds inside a chunk) and beta up to 2
    (allow_neg_eigval): nothing overflows, and both kernels agree with the formulas."""
    q, k, v, g, beta, _ = synth_gdn_inputs(1, 256, 2, 128, 128, seed=11)
    g = g * 6.0
    beta = (beta.float() * 2.0).bfloat16()
    ref = _reference(q, k, v, g, beta)
    for kernel in ("natsl_gdn_chunk_prep_tc", "natsl_gdn_chunk_prep_ex"):
        got = _run(kernel, q, k, v, g, beta, True)
        for i, n in enumerate(("gcs", "k_rstd", "q_rstd", "w", "u", "P")):
            _check(got[i], ref[i], f"{kernel}: {n}", 2e-5 if i < 3 else 2e-2)


def test_prep_tc_is_bit_reproducible_and_close_to_the_mma_sync_kernel():
    q, k, v, g, beta, _ = synth_gdn_inputs(2, 1024, 4, 128, 128, seed=5)
    a = _run("natsl_gdn_chunk_prep_tc", q, k, v, g, beta, True)
    b = _run("natsl_gdn_chunk_prep_tc", q, k, v, g, beta, True)
    c = _run("natsl_gdn_chunk_prep_ex", q, k, v, g, beta, True)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    assert torch.equal(a[0], c[0])                          # the cumsum is the same tree in both kernels
    for i, n in enumerate(("gcs", "k_rstd", "q_rstd", "w", "u", "P")):
        _check(a[i], c[i].double().cpu(), f"tc vs mma.sync: {n}", 2e-5 if i < 3 else 1e-2)


def test_prep_tc_refuses_other_head_dims():
    from neuralattentionsearchlinear_b200 import _lib
    q, k, v, g, beta, _ = synth_gdn_inputs(1, 64, 1, 64, 64, seed=1)
    with pytest.raises(_lib.NatslError):
        _run("natsl_gdn_chunk_prep_tc", q, k, v, g, beta, True)
