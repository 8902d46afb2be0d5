"""GPU parity tests of the backward pass (-m gpu): the CUDA kernels, called through the C ABI, against the CPU oracle
(``oracle/grad.py``) evaluated in float64 on the same bf16-rounded inputs.

Tolerance: |got - ref| <= 1e-2 |ref| + 1e-2 s — the forward's rtol = atol = 1e-2 with the absolute part scaled to the
size of the gradient (see ``close_scaled``); gradients are sums over many tokens and are not O(1)."""
import pytest
import torch

from oracle import attn as oattn
from oracle import gdn as ogdn
from oracle import grad as ograd
from oracle import tables as otab
from tests.helpers import synth_gdn_inputs, synth_mamba_inputs

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def nat():
    import neuralattentionsearchlinear_b200 as n
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return n


def close_scaled(got, ref, what, tol=TOL, scale="auto"):
    """|got - ref| <= tol |ref| + tol s.  A gradient vector is a sum of many bf16 products whose rounding error grows
    with the size of the terms, not of the result, so the absolute part is scaled: for [..., D] vectors (ndim >= 4) by
    the largest entry of the same vector, for per-token scalars by the spread of the tensor, for block sums
    (``scale='max'``: dnats, sums of score gradients over thousands of (query, key) pairs that largely cancel) by the
    largest entry of the tensor; never below 1 (the forward's atol)."""
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    if scale == "max":
        s = ref.abs().max().clamp_min(1.0)
    elif ref.dim() >= 4:
        s = ref.abs().amax(-1, keepdim=True).clamp_min(1.0)
    else:
        s = torch.tensor(max(1.0, float(ref.std())) if ref.numel() > 1 else 1.0)
    err = (got - ref).abs()
    bad = err > tol * ref.abs() + tol * s
    assert not bad.any(), (f"{what}: {int(bad.sum())}/{bad.numel()} outside tolerance; max abs err {err.max().item():.4g}, "
                           f"ref max {ref.abs().max().item():.4g}, ref std {float(ref.std()):.4g}")


# ------------------------------------------------------------------------------------------------ softmax branch
@pytest.mark.parametrize("B,T,HQ,HKV,HN,DK,DV,nbs,own,compat", [
    (2, 512, 4, 4, 4, 64, 64, 64, True, False),          # the CPU configuration's head shape
    (1, 704, 4, 2, 2, 128, 128, 64, True, False),        # two query heads per key/value head
    (2, 1024, 2, 2, 2, 64, 128, 128, True, False),       # block 128: own block spans two tiles
    (1, 1100, 2, 2, 1, 128, 64, 256, True, False),       # ragged last tile, one selection head for two heads
    (2, 512, 4, 4, 4, 64, 64, 64, False, False),         # softmax branch without the own block
    (2, 512, 4, 2, 2, 128, 128, 64, True, True),         # the reference's default backward (own-block terms dropped)
])
def test_attention_backward(nat, B, T, HQ, HKV, HN, DK, DV, nbs, own, compat):
    from neuralattentionsearchlinear_b200 import _lib, _ops
    gen = torch.Generator().manual_seed(T + DK + nbs)
    q = torch.randn(B, T, HQ, DK, generator=gen).bfloat16()
    k = torch.randn(B, T, HKV, DK, generator=gen).bfloat16()
    v = torch.randn(B, T, HKV, DV, generator=gen).bfloat16()
    do = torch.randn(B, T, HQ, DV, generator=gen).bfloat16()
    types = otab.synth_types(B, -(-T // nbs), HN, 0.3, seed=T)
    tb = nat.build_selection_tables(types.cuda(), T, nbs)
    scale = DK ** -0.5
    o, lse = _ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), tb, scale, own)
    dq, dk, dv, dnats = _ops.attn_bwd(q.cuda(), k.cuda(), v.cuda(), o, lse, do.cuda(), tb, scale, own, reference_compat=compat)
    ref = ograd.attn_grads(q.double(), k.double(), v.double(), types[..., 0], do.double(), nbs=nbs, scale=scale,
                           own_chunk=own, reference_compat=compat)
    close_scaled(dq, ref["dq"], "dq")
    close_scaled(dk, ref["dk"], "dk")
    close_scaled(dv, ref["dv"], "dv")
    close_scaled(dnats, ref["dnats"], "dnats (softmax column)", scale="max")
    assert _lib.load().natsl_device_status() == 0
    # deterministic: no atomics on global memory
    dq2, dk2, dv2, dn2 = _ops.attn_bwd(q.cuda(), k.cuda(), v.cuda(), o, lse, do.cuda(), tb, scale, own, reference_compat=compat)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2) and torch.equal(dnats, dn2)


# ------------------------------------------------------------------------------------------------ linear branch
def _linear_case(nat, rule, B, T, H, HN, K, V, seed, use_h0, decay, p_sel=0.6, invalid=True):
    from neuralattentionsearchlinear_b200 import _lib, _ops
    gdn = rule == "gdn"
    if gdn:
        q, k, v, g, beta, h0 = synth_gdn_inputs(B, T, H, K, V, seed=seed, normalize_qk=False)
    else:
        q, k, v, g, h0 = synth_mamba_inputs(B, T, H, K, V, seed=seed)
        beta = None
    NT = -(-T // 64)
    types = otab.synth_types(B, NT, HN, 1.0 - p_sel, seed=seed + 1)
    gen = torch.Generator().manual_seed(seed + 2)
    do = torch.randn(B, T, H, V, generator=gen).bfloat16()
    dht = torch.randn(B, H, K, V, generator=gen) * 0.1
    h0 = h0 if use_h0 else None
    scale = K ** -0.5 if gdn else 1.0
    dev = torch.device("cuda")
    tb = nat.build_selection_tables(types.to(dev), T, 64)
    c = lambda x: None if x is None else x.to(dev)
    out = _ops.linear_bwd(_lib.RULE_GDN if gdn else _lib.RULE_MAMBA, c(q), c(k), c(v), c(g), c(beta), tb, scale, c(h0),
                          decay, gdn, c(do), dht=c(dht), invalid_dnats=invalid, return_intermediates=True)
    assert _lib.load().natsl_device_status() == 0
    d = lambda x: None if x is None else x.double()
    kw = dict(scale=scale, h0=d(h0), decay=decay, use_l2norm=gdn, rule=rule)
    return out, (d(q), d(k), d(v), d(g), d(beta), types[..., 1], d(do), d(dht)), kw


@pytest.mark.parametrize("rule,B,T,H,HN,K,V,use_h0,decay", [
    ("gdn", 2, 512, 4, 4, 64, 64, False, True),           # the CPU configuration's shape
    ("gdn", 1, 512, 2, 2, 128, 128, True, True),          # the benchmark's head dims, initial state
    ("gdn", 2, 256, 4, 2, 128, 64, True, False),          # K != V, two heads per selection head, no decay over skipped blocks
    ("gdn", 1, 384, 2, 2, 64, 128, False, True),
    ("mamba", 2, 512, 4, 4, 128, 64, True, True),         # Mamba2 / SSD rule at the long-context head shape
    ("mamba", 1, 256, 2, 1, 64, 64, False, False),
])
def test_linear_backward_whole_chunks(nat, rule, B, T, H, HN, K, V, use_h0, decay):
    out, (q, k, v, g, beta, sel, do, dht), kw = _linear_case(nat, rule, B, T, H, HN, K, V, seed=K + V + T, use_h0=use_h0,
                                                            decay=decay)
    ref = ograd.linear_chunk_backward(q, k, v, g, beta, sel, do, dht, **kw)
    # intermediates first: they localise a failure
    selh = ogdn._expand_sel(sel, H)                                        # [B,NT,H]
    m = selh[..., None, None]                                              # only updating chunks are stored
    close_scaled(torch.where(m, out["dS"].double().cpu(), torch.zeros(())), torch.where(m, ref["dS"], torch.zeros(())),
                 "dS (state gradient after updating chunks)")
    close_scaled(out["dvp"], ref["dvp"], "dv'")
    if rule == "gdn":
        close_scaled(out["dw"], ref["dw"], "dw")
    close_scaled(out["dv"], ref["dv"], "dv")
    close_scaled(out["dq"], ref["dq"], "dq")
    close_scaled(out["dk"], ref["dk"], "dk")
    close_scaled(out["dg"], ref["dg"], "dg")
    if rule == "gdn":
        close_scaled(out["dbeta"], ref["dbeta"], "dbeta")
    if use_h0:
        close_scaled(out["dh0"], ref["dh0"], "dh0")
    dn_ref = ograd.dnats_linear(q, k, v, g, beta, sel, do, dht, invalid_blocks=True, **kw)
    close_scaled(out["dnats"], dn_ref, "dnats (linear column)", scale="max")
    # run-to-run bit-identity (every reduction has a fixed order)
    out2, _, _ = _linear_case(nat, rule, B, T, H, HN, K, V, seed=K + V + T, use_h0=use_h0, decay=decay)
    for name in ("dq", "dk", "dv", "dg", "dnats"):
        assert torch.equal(out[name], out2[name]), f"{name} differs between two runs"


def test_linear_backward_against_autograd_ragged(nat):
    """Ragged last chunk (T = 300): against autograd through the token recurrence with re-roll (the oracle's normative
    form), which takes any length."""
    from neuralattentionsearchlinear_b200 import _lib, _ops
    B, T, H, HN, K, V = 2, 300, 2, 2, 64, 64
    q, k, v, g, beta, h0 = synth_gdn_inputs(B, T, H, K, V, seed=11, normalize_qk=False)
    NT = -(-T // 64)
    types = otab.synth_types(B, NT, HN, 0.4, seed=12)
    gen = torch.Generator().manual_seed(13)
    do = torch.randn(B, T, H, V, generator=gen).bfloat16()
    dev = torch.device("cuda")
    tb = nat.build_selection_tables(types.to(dev), T, 64)
    scale = K ** -0.5
    out = _ops.linear_bwd(_lib.RULE_GDN, q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), tb, scale, h0.to(dev),
                          True, True, do.to(dev), dht=None)
    ref = ograd.linear_true_grads(q.double(), k.double(), v.double(), g.double(), beta.double(), types[..., 1], do.double(),
                                  None, scale=scale, h0=h0.double(), decay=True, use_l2norm=True, rule="gdn")
    for name in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
        close_scaled(out[name], ref[name], name)


def test_linear_backward_selected_only_dnats(nat):
    out, (q, k, v, g, beta, sel, do, dht), kw = _linear_case(nat, "gdn", 1, 512, 2, 2, 64, 64, seed=5, use_h0=False,
                                                            decay=True, invalid=False)
    dn_ref = ograd.dnats_linear(q, k, v, g, beta, sel, do, dht, invalid_blocks=False, **kw)
    close_scaled(out["dnats"], dn_ref, "dnats (linear column, selected blocks only)", scale="max")


# ------------------------------------------------------------------------------------------------ the ops under autograd
@pytest.mark.parametrize("K,V,mode", [(64, 64, "all"), (128, 128, "all"), (128, 128, "gated_delta_net")])
def test_gdn_op_autograd(nat, K, V, mode):
    """loss.backward() through nats_mixed_attn_gdn: gradients of every differentiable input, and dnats."""
    B, T, H = 2, 512, 4
    q, k, v, g, beta, h0 = synth_gdn_inputs(B, T, H, K, V, seed=K, normalize_qk=False)
    types = otab.synth_types(B, T // 64, H, 0.3, seed=K + 1)
    gen = torch.Generator().manual_seed(K + 2)
    do_l = torch.randn(B, T, H, V, generator=gen).bfloat16()
    do_a = torch.randn(B, T, H, V, generator=gen).bfloat16()
    dev = torch.device("cuda")
    leaf = lambda x: x.to(dev).requires_grad_(True)
    qa, ka, va, ql, kl, vl, gg, bb, ty = (leaf(x) for x in (q, k, v, q, k, v, g, beta, types))
    o_l, o_a, ht = nat.nats_mixed_attn_gdn(qa, ka, va, ql, kl, vl, None, gg, bb, ty, None, nats_block_size=64,
                                           ops_for_incomplete_chunks=mode, output_final_state_gated_delta=True,
                                           decay_for_non_gdn_blocks=True)
    assert o_l.requires_grad and o_a.requires_grad
    loss = (o_l.float() * do_l.to(dev).float()).sum() + (o_a.float() * do_a.to(dev).float()).sum()
    loss.backward()
    own = mode == "all"
    ra = ograd.attn_grads(q.double(), k.double(), v.double(), types[..., 0], do_a.double(), nbs=64, own_chunk=own)
    rl = ograd.linear_chunk_backward(q.double(), k.double(), v.double(), g.double(), beta.double(), types[..., 1],
                                     do_l.double(), None, decay=True)
    close_scaled(qa.grad, ra["dq"], "dq_attn")
    close_scaled(ka.grad, ra["dk"], "dk_attn")
    close_scaled(va.grad, ra["dv"], "dv_attn")
    close_scaled(ql.grad, rl["dq"], "dq_lattn")
    close_scaled(kl.grad, rl["dk"], "dk_lattn")
    close_scaled(vl.grad, rl["dv"], "dv_lattn")
    close_scaled(gg.grad, rl["dg"], "dg")
    close_scaled(bb.grad, rl["dbeta"], "dbeta")
    dn_l = ograd.dnats_linear(q.double(), k.double(), v.double(), g.double(), beta.double(), types[..., 1], do_l.double(),
                              None, invalid_blocks=True, decay=True)
    close_scaled(ty.grad[..., 0], ra["dnats"], "dnats column 0", scale="max")
    close_scaled(ty.grad[..., 1], dn_l, "dnats column 1", scale="max")


def test_mamba_op_autograd(nat):
    B, T, H, K, V = 1, 512, 4, 128, 64
    q, k, v, g, h0 = synth_mamba_inputs(B, T, H, K, V, seed=3)
    types = otab.synth_types(B, T // 64, H, 0.2, seed=4)
    gen = torch.Generator().manual_seed(5)
    do_l = torch.randn(B, T, H, V, generator=gen).bfloat16()
    dev = torch.device("cuda")
    leaf = lambda x: x.to(dev).requires_grad_(True)
    ql, kl, vl, gg = (leaf(x) for x in (q, k, v, g))
    o_l, o_a, _ = nat.nats_mixed_attn_mamba(ql, kl, vl, ql, kl, vl, None, gg, types.to(dev), None, scale_attn=K ** -0.5,
                                            nats_block_size=64, ops_for_incomplete_chunks="all",
                                            decay_for_non_mamba_blocks=True)
    (o_l.float() * do_l.to(dev).float()).sum().backward()
    rl = ograd.linear_chunk_backward(q.double(), k.double(), v.double(), g.double(), None, types[..., 1], do_l.double(),
                                     None, scale=1.0, decay=True, use_l2norm=False, rule="mamba")
    close_scaled(ql.grad, rl["dq"], "dq")
    close_scaled(kl.grad, rl["dk"], "dk")
    close_scaled(vl.grad, rl["dv"], "dv")
    close_scaled(gg.grad, rl["dg"], "dg")


def test_reference_compat_switch(nat):
    """Inside ``reference_compat_bwd()`` the op's softmax-branch gradients are the reference's (own-block terms dropped)."""
    from neuralattentionsearchlinear_b200 import mixed_attn_gdn as m
    B, T, H, K = 1, 256, 2, 64
    q, k, v, g, beta, _ = synth_gdn_inputs(B, T, H, K, K, seed=21, normalize_qk=False)
    types = otab.synth_types(B, T // 64, H, 0.4, seed=22)
    do_a = torch.randn(B, T, H, K, generator=torch.Generator().manual_seed(23)).bfloat16()
    dev = torch.device("cuda")
    qa = q.to(dev).requires_grad_(True)
    with m.reference_compat_bwd():
        _, o_a, _ = nat.nats_mixed_attn_gdn(qa, k.to(dev), v.to(dev), q.to(dev), k.to(dev), v.to(dev), None, g.to(dev),
                                            beta.to(dev), types.to(dev), None, ops_for_incomplete_chunks="all")
    (o_a.float() * do_a.to(dev).float()).sum().backward()
    ref = ograd.attn_grads(q.double(), k.double(), v.double(), types[..., 0], do_a.double(), reference_compat=True)
    close_scaled(qa.grad, ref["dq"], "dq_attn (reference-compatible)")


def test_backward_raises_where_not_built(nat):
    """fp32 tensors and block sizes other than 64 run forward only: backward raises instead of returning nothing."""
    B, T, H, K = 1, 256, 2, 64
    q, k, v, g, beta, _ = synth_gdn_inputs(B, T, H, K, K, seed=31, dtype=torch.float32)
    types = otab.synth_types(B, T // 64, H, 0.4, seed=32)
    dev = torch.device("cuda")
    qa = q.to(dev).requires_grad_(True)
    o_l, _, _ = nat.nats_mixed_attn_gdn(qa, k.to(dev), v.to(dev), qa, k.to(dev), v.to(dev), None, g.to(dev), beta.to(dev),
                                        types.to(dev), None, ops_for_incomplete_chunks="all")
    with pytest.raises(NotImplementedError):
        o_l.sum().backward()
    qb = q.bfloat16().to(dev).requires_grad_(True)
    types128 = otab.synth_types(B, T // 128, H, 0.4, seed=33)
    o_l, _, _ = nat.nats_mixed_attn_gdn(qb, k.bfloat16().to(dev), v.bfloat16().to(dev), qb, k.bfloat16().to(dev),
                                        v.bfloat16().to(dev), None, g.to(dev), beta.bfloat16().to(dev), types128.to(dev), None,
                                        nats_block_size=128, ops_for_incomplete_chunks="all")
    with pytest.raises(NotImplementedError):
        o_l.float().sum().backward()


# ------------------------------------------------------------------------------------------------ output mixing
@pytest.mark.parametrize("D,act,with_w", [(128, "swish", True), (64, "sigmoid", True), (256, "swish", False)])
def test_norm_gate_backward(nat, D, act, with_w):
    from neuralattentionsearchlinear_b200.modules import FusedMultiInputRMSNormGated
    rows = 3 * 100 * 4
    gen = torch.Generator().manual_seed(D)
    x1 = torch.randn(3, 100, 4, D, generator=gen).bfloat16()
    x2 = (torch.randn(3, 100, 4, D, generator=gen) * 2).bfloat16()
    g = torch.randn(3, 100, 4, D, generator=gen).bfloat16()
    xw = torch.rand(3, 100, 4, 2, generator=gen).softmax(-1) if with_w else None
    dy = torch.randn(3, 100, 4, D, generator=gen).bfloat16()
    dev = torch.device("cuda")
    mod = FusedMultiInputRMSNormGated(D, eps=1e-5, activation=act).to(dev)
    with torch.no_grad():
        mod.weight1.copy_(1 + 0.1 * torch.randn(D, generator=gen))
        mod.weight2.copy_(1 + 0.1 * torch.randn(D, generator=gen))
    leaf = lambda t: None if t is None else t.to(dev).requires_grad_(True)
    a, b, c, w = leaf(x1), leaf(x2), leaf(g), leaf(xw)
    y = mod(a, b, c, w)
    (y.float() * dy.to(dev).float()).sum().backward()
    # the same expression in float64 on the CPU
    A, Bv, Cg = x1.double().requires_grad_(True), x2.double().requires_grad_(True), g.double().requires_grad_(True)
    W = None if xw is None else xw.double().requires_grad_(True)
    w1 = mod.weight1.detach().double().cpu().requires_grad_(True)
    w2 = mod.weight2.detach().double().cpu().requires_grad_(True)
    rms = lambda x: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)
    m1 = 1.0 if W is None else W[..., :1]
    m2 = 1.0 if W is None else W[..., 1:]
    vv = rms(A) * w1 * m1 + rms(Bv) * w2 * m2
    yy = vv * (torch.sigmoid(Cg) if act == "sigmoid" else Cg * torch.sigmoid(Cg))
    (yy * dy.double()).sum().backward()
    close_scaled(y, yy, "y")
    close_scaled(a.grad, A.grad, "dx1")
    close_scaled(b.grad, Bv.grad, "dx2")
    close_scaled(c.grad, Cg.grad, "dg")
    close_scaled(mod.weight1.grad, w1.grad, "dw1")
    close_scaled(mod.weight2.grad, w2.grad, "dw2")
    if with_w:
        close_scaled(w.grad, W.grad, "d(mixing weights)")
    assert rows == a.grad.numel() // D
