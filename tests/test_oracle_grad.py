"""The backward oracle (oracle/grad.py) against independent evaluations on CPU in float64: the two forms of the
linear branch give the same gradients; the closed forms of the reference's ``dnats`` columns equal the autograd
derivatives they stand for; the attention gradients equal autograd through the forward oracle."""
import pytest
import torch

from oracle import attn as oattn
from oracle import gdn as ogdn
from oracle import grad as ograd
from oracle import tables as otab

DT = torch.float64


def _inputs(B, T, H, K, V, seed):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=gen, dtype=DT)
    k = torch.randn(B, T, H, K, generator=gen, dtype=DT)
    v = torch.randn(B, T, H, V, generator=gen, dtype=DT)
    g = -torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen, dtype=DT)) * 0.3
    beta = torch.randn(B, T, H, generator=gen, dtype=DT).sigmoid()
    do = torch.randn(B, T, H, V, generator=gen, dtype=DT)
    dht = torch.randn(B, H, K, V, generator=gen, dtype=DT)
    h0 = torch.randn(B, H, K, V, generator=gen, dtype=DT) * 0.1
    return q, k, v, g, beta, do, dht, h0


@pytest.mark.parametrize("rule", ["gdn", "mamba"])
@pytest.mark.parametrize("decay", [True, False])
def test_probe_form_equals_chunk_oracle_and_its_gradients_equal_the_recurrent_form(rule, decay):
    B, T, H, K, V = 2, 256, 2, 8, 6
    q, k, v, g, beta, do, dht, h0 = _inputs(B, T, H, K, V, 1)
    types = otab.synth_types(B, T // 64, 2, 0.5, seed=2, dtype=DT)
    types[:, -1] = 1
    sel = types[..., 1]
    kw = dict(scale=0.5, decay=decay, use_l2norm=(rule == "gdn"), rule=rule)
    o_ref, s_ref = ogdn.linear_chunk(q, k, v, g, beta, sel, nbs=64, h0=h0, reference_trailing_carry=False, **kw)
    leaves = [x.detach().clone().requires_grad_(True) for x in (q, k, v, g, beta, h0)]
    o, sfin, _, _ = ograd.chunk_forward_with_probes(leaves[0], leaves[1], leaves[2], leaves[3],
                                                    leaves[4] if rule == "gdn" else None, sel, h0=leaves[5], **kw)
    assert (o - o_ref).abs().max() < 1e-10 and (sfin - s_ref).abs().max() < 1e-10
    ((o * do).sum() + (sfin * dht).sum()).backward()
    true = ograd.linear_true_grads(q, k, v, g, beta, sel, do, dht, h0=h0, **kw)
    names = ["dq", "dk", "dv", "dg", "dbeta", "dh0"]
    for n, leaf in zip(names, leaves):
        if n == "dbeta" and rule != "gdn":
            continue
        assert (leaf.grad - true[n]).abs().max() < 1e-8, n


@pytest.mark.parametrize("rule", ["gdn", "mamba"])
def test_dnats_linear_is_the_gate_derivative_on_selected_blocks(rule):
    B, T, H, K, V = 1, 320, 4, 8, 4
    q, k, v, g, beta, do, dht, _ = _inputs(B, T, H, K, V, 3)
    types = otab.synth_types(B, T // 64, 2, 0.5, seed=4, dtype=DT)
    types[:, -1] = 1
    sel = types[..., 1]
    kw = dict(scale=0.7, decay=True, use_l2norm=(rule == "gdn"), rule=rule)
    b = beta if rule == "gdn" else None
    got = ograd.dnats_linear(q, k, v, g, b, sel, do, dht, invalid_blocks=False, **kw)          # [B,NT,HN]
    gate = torch.ones(B, T // 64, H, dtype=DT, requires_grad=True)
    o, sfin, _, _ = ograd.chunk_forward_with_probes(q, k, v, g, b, sel, write_gate=gate, **kw)
    ((o * do).sum() + (sfin * dht).sum()).backward()
    want = torch.where(ogdn._expand_sel(sel, H), gate.grad, torch.zeros_like(gate.grad)).view(B, T // 64, 2, 2).sum(-1)
    assert (got - want).abs().max() < 1e-9
    # with the flag for the other blocks: same values on selected blocks, something finite elsewhere, zero after the
    # last selected block
    full = ograd.dnats_linear(q, k, v, g, b, sel, do, dht, invalid_blocks=True, **kw)
    m = sel.to(torch.bool)
    assert (full[m] - got[m]).abs().max() < 1e-12 and torch.isfinite(full).all()


@pytest.mark.parametrize("own_chunk", [True, False])
def test_attention_gradients_equal_autograd(own_chunk):
    B, T, HQ, HKV, K, V, nbs = 2, 256, 4, 2, 8, 6, 64
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(B, T, HQ, K, generator=gen, dtype=DT)
    k = torch.randn(B, T, HKV, K, generator=gen, dtype=DT)
    v = torch.randn(B, T, HKV, V, generator=gen, dtype=DT)
    do = torch.randn(B, T, HQ, V, generator=gen, dtype=DT)
    types = otab.synth_types(B, T // nbs, 2, 0.5, seed=6, dtype=DT)
    sel = types[..., 0]
    got = ograd.attn_grads(q, k, v, sel, do, nbs=nbs, scale=0.4, own_chunk=own_chunk)
    ql, kl, vl = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
    mask = oattn.attn_mask(sel, T, nbs, HQ, own_chunk=own_chunk)
    o, _ = oattn.attn_sdpa(ql, kl, vl, mask, 0.4)
    (o * do).sum().backward()
    for n, leaf in (("dq", ql), ("dk", kl), ("dv", vl)):
        assert (got[n] - leaf.grad).abs().max() < 1e-10, n
    compat = ograd.attn_grads(q, k, v, sel, do, nbs=nbs, scale=0.4, own_chunk=own_chunk, reference_compat=True)
    if not own_chunk:                                       # nothing to drop: the reference's form is the true gradient
        for n in ("dq", "dk", "dv"):
            assert (compat[n] - got[n]).abs().max() < 1e-12
    else:
        assert (compat["dk"] - got["dk"]).abs().max() > 1e-3   # the own-chunk terms are really gone


def test_dnats_attn_is_the_bias_derivative_on_selected_blocks():
    B, T, HQ, HKV, K, V, nbs = 1, 256, 4, 4, 8, 4, 64
    gen = torch.Generator().manual_seed(7)
    q = torch.randn(B, T, HQ, K, generator=gen, dtype=DT)
    k = torch.randn(B, T, HKV, K, generator=gen, dtype=DT)
    v = torch.randn(B, T, HKV, V, generator=gen, dtype=DT)
    do = torch.randn(B, T, HQ, V, generator=gen, dtype=DT)
    types = otab.synth_types(B, T // nbs, 2, 0.6, seed=8, dtype=DT)
    sel = types[..., 0]
    got = ograd.attn_grads(q, k, v, sel, do, nbs=nbs, scale=0.4)["dnats"]                       # [B,TN,HN]
    # additive bias per (block, head) on the scaled scores of the block's keys for the queries of later blocks
    TN = T // nbs
    bias = torch.zeros(B, HQ, TN, dtype=DT, requires_grad=True)
    mask = oattn.attn_mask(sel, T, nbs, HQ)
    blk = torch.arange(T) // nbs
    past = (torch.arange(T)[:, None] >= (blk[None, :] + 1) * nbs)[None, None]
    s = (q.permute(0, 2, 1, 3) @ k.permute(0, 2, 1, 3).transpose(-1, -2)) * 0.4
    s = s + torch.where(past, bias[:, :, blk][:, :, None, :].expand(B, HQ, T, T), torch.zeros((), dtype=DT))
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
    o = (p @ v.permute(0, 2, 1, 3)).permute(0, 2, 1, 3)
    (o * do).sum().backward()
    want = bias.grad.view(B, 2, 2, TN).sum(2).permute(0, 2, 1)
    want = torch.where(sel.to(torch.bool), want, torch.zeros_like(want))
    assert (got - want).abs().max() < 1e-10


@pytest.mark.parametrize("rule", ["gdn", "mamba"])
@pytest.mark.parametrize("decay,use_h0", [(True, True), (False, False)])
def test_written_out_chunk_backward_equals_autograd(rule, decay, use_h0):
    B, T, H, K, V = 2, 320, 2, 8, 6
    q, k, v, g, beta, do, dht, h0 = _inputs(B, T, H, K, V, 9)
    types = otab.synth_types(B, T // 64, 2, 0.5, seed=10, dtype=DT)
    types[0, -1] = 1                                        # batch 0 ends selected, batch 1 as drawn
    sel = types[..., 1]
    kw = dict(scale=0.6, decay=decay, use_l2norm=(rule == "gdn"), rule=rule, h0=h0 if use_h0 else None)
    b = beta if rule == "gdn" else None
    got = ograd.linear_chunk_backward(q, k, v, g, b, sel, do, dht, **kw)
    true = ograd.linear_true_grads(q, k, v, g, beta, sel, do, dht, **kw)
    for n in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
        if true[n] is None:
            assert got[n] is None
            continue
        assert (got[n] - true[n]).abs().max() < 1e-8, (n, float((got[n] - true[n]).abs().max()))


def test_state_gradients_of_the_written_out_backward_equal_the_probe_gradients():
    B, T, H, K, V = 1, 320, 2, 8, 6
    q, k, v, g, beta, do, dht, h0 = _inputs(B, T, H, K, V, 11)
    types = otab.synth_types(B, T // 64, 2, 0.5, seed=12, dtype=DT)
    types[:, -1] = 1
    sel = types[..., 1]
    kw = dict(scale=0.6, decay=True, use_l2norm=True, rule="gdn", h0=h0)
    got = ograd.linear_chunk_backward(q, k, v, g, beta, sel, do, dht, **kw)
    o, sfin, probes, _ = ograd.chunk_forward_with_probes(q, k, v, g, beta, sel, **kw)
    grads = torch.autograd.grad((o * do).sum() + (sfin * dht).sum(), probes, allow_unused=True)
    for c, gr in enumerate(grads):
        want = torch.zeros_like(got["dS"][:, c]) if gr is None else gr
        # the probe sits after the chunk and after the point where the final state is taken, so on the last
        # selected chunk it also receives the gradient of the final state, like dS
        assert (got["dS"][:, c] - want).abs().max() < 1e-9, c


def test_regression_pin_of_the_no_own_chunk_mode_and_the_backward_oracle():
    """tests/golden/oracle_grad_pin.npz (written by tests/golden/make_golden.py) pins the oracle's own values."""
    import importlib.util
    import os
    import numpy as np
    golden_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(golden_dir, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    z = np.load(os.path.join(golden_dir, "oracle_grad_pin.npz"))
    x = mg.grad_pin_inputs()
    sel = x["types"][..., 1]
    o_na, s_na = ogdn.linear_chunk(x["q"], x["k"], x["v"], x["g"], x["beta"], sel, nbs=64, own_chunk=False)
    assert np.allclose(o_na[:, ::5].numpy(), z["o_no_own"], atol=1e-12) and np.allclose(s_na.numpy(), z["s_no_own"], atol=1e-12)
    gr = ograd.linear_chunk_backward(x["q"], x["k"], x["v"], x["g"], x["beta"], sel, x["do"], x["dht"], decay=True)
    for n in ("dq", "dk", "dv"):
        assert np.allclose(gr[n][:, ::5].numpy(), z[n], atol=1e-10), n
    assert np.allclose(gr["dg"].numpy(), z["dg"], atol=1e-10) and np.allclose(gr["dbeta"].numpy(), z["dbeta"], atol=1e-10)
    dn = ograd.dnats_linear(x["q"], x["k"], x["v"], x["g"], x["beta"], sel, x["do"], x["dht"], decay=True)
    assert np.allclose(dn.numpy(), z["dnats_lin"], atol=1e-10)
    ga = ograd.attn_grads(x["q"], x["k"], x["v"], x["types"][..., 0], x["do"], nbs=64, reference_compat=True)
    assert np.allclose(ga["dq"][:, ::5].numpy(), z["dq_attn_compat"], atol=1e-10)
    assert np.allclose(ga["dk"][:, ::5].numpy(), z["dk_attn_compat"], atol=1e-10)
    assert np.allclose(ga["dnats"].numpy(), z["dnats_attn"], atol=1e-10)
