"""Oracle self-consistency and pins: token recurrence with re-roll vs chunk form,
third-party naive GDN (all blocks selected), softmax mask/SDPA, regression pin."""
import os

import numpy as np
import pytest
import torch

from oracle import attn as oattn
from oracle import gdn as ogdn
from oracle import mamba as omamba
from oracle import tables as otab


def _inputs(B, T, H, K, V, seed, dtype=torch.float64):
    g_ = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=g_, dtype=dtype)
    k = torch.randn(B, T, H, K, generator=g_, dtype=dtype)
    v = torch.randn(B, T, H, V, generator=g_, dtype=dtype)
    beta = torch.randn(B, T, H, generator=g_, dtype=dtype).sigmoid()
    g = -torch.nn.functional.softplus(torch.randn(B, T, H, generator=g_, dtype=dtype))
    h0 = torch.randn(B, H, K, V, generator=g_, dtype=dtype)
    return q, k, v, g, beta, h0


@pytest.mark.parametrize("nbs,decay,T,HN", [(64, True, 512, 4), (64, False, 320, 2), (128, True, 512, 4),
                                            (256, True, 600, 1), (64, True, 200, 4), (64, True, 64, 4)])
@pytest.mark.parametrize("rule", ["gdn", "mamba"])
def test_recurrent_equals_chunk(nbs, decay, T, HN, rule):
    B, H, K, V = 2, 4, 16, 24
    q, k, v, g, beta, h0 = _inputs(B, T, H, K, V, seed=T + nbs)
    ty = otab.synth_types(B, -(-T // nbs), HN, 0.4, seed=1)
    kw = dict(nbs=nbs, h0=h0, decay=decay, rule=rule, use_l2norm=(rule == "gdn"))
    o1, s1 = ogdn.linear_recurrent(q, k, v, g, beta, ty[..., 1], **kw)
    o2, s2 = ogdn.linear_chunk(q, k, v, g, beta, ty[..., 1], **kw)
    assert (o1 - o2).abs().max() < 1e-11
    assert (s1 - s2).abs().max() < 1e-11


def test_trailing_carry_quirk_only_matters_after_last_selected():
    B, T, H, K, V = 1, 320, 1, 8, 8
    q, k, v, g, beta, h0 = _inputs(B, T, H, K, V, seed=3)
    sel = torch.tensor([1, 0, 1, 0, 0]).view(1, 5, 1)
    a, _ = ogdn.linear_chunk(q, k, v, g, beta, sel, h0=h0, reference_trailing_carry=True)
    b, _ = ogdn.linear_chunk(q, k, v, g, beta, sel, h0=h0, reference_trailing_carry=False)
    r, _ = ogdn.linear_recurrent(q, k, v, g, beta, sel, h0=h0)
    assert torch.equal(a[:, :256], b[:, :256])            # up to the first trailing skipped block: identical
    assert (b - r).abs().max() < 1e-12                      # the normative recurrence carries on
    assert (a[:, 256:] - b[:, 256:]).abs().max() > 1e-6     # the reference's chunk kernels do not


def test_gdn_against_third_party_naive(golden_dir):
    z = np.load(os.path.join(golden_dir, "gdn_fla_naive.npz"))
    t = {k: torch.from_numpy(z[k]).double() for k in z.files}
    B, T, H, K = t["q"].shape
    sel = torch.ones(B, -(-T // 64), H)
    # the third-party function does not normalise q/k: compare with use_l2norm=False
    o, s = ogdn.linear_chunk(t["q"], t["k"], t["v"], t["g"], t["beta"], sel, h0=t["h0"], use_l2norm=False)
    assert (o - t["o"]).abs().max() < 2e-5
    assert (s - t["s"]).abs().max() < 2e-5
    o, s = ogdn.linear_recurrent(t["q"], t["k"], t["v"], t["g"], t["beta"], sel, h0=t["h0"], use_l2norm=False)
    assert (o - t["o"]).abs().max() < 2e-5


def test_mask_formula_small():
    sel = torch.tensor([1, 0, 1, 0]).view(1, 4, 1)
    m = oattn.attn_mask(sel, 16, 4, 1)[0, 0]
    for t in range(16):
        for s in range(16):
            cs, ct = s // 4, t // 4
            exp = (sel[0, cs, 0] == 1 and t >= (cs + 1) * 4) or (cs == ct and s <= t)
            assert bool(m[t, s]) == bool(exp)
    m2 = oattn.attn_mask(sel, 16, 4, 1, own_chunk=False)[0, 0]
    assert not m2[:4].any() and bool(m2[4, 0]) and not bool(m2[8, 4])


def test_sdpa_matches_torch():
    g_ = torch.Generator().manual_seed(0)
    B, T, HQ, HKV, K, V = 2, 200, 4, 2, 16, 24
    q = torch.randn(B, T, HQ, K, generator=g_)
    k = torch.randn(B, T, HKV, K, generator=g_)
    v = torch.randn(B, T, HKV, V, generator=g_)
    ty = otab.synth_types(B, 4, 2, 0.5, seed=2)
    mask = oattn.attn_mask(ty[..., 0], T, 64, HQ)
    o, lse = oattn.attn_sdpa(q, k, v, mask)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(2, 1), v.transpose(1, 2).repeat_interleave(2, 1),
        attn_mask=mask).transpose(1, 2)
    assert (o - ref).abs().max() < 1e-5
    # no-key rows (own_chunk=False) give zeros
    mask0 = oattn.attn_mask(ty[..., 0], T, 64, HQ, own_chunk=False)
    o0, lse0 = oattn.attn_sdpa(q, k, v, mask0)
    assert torch.equal(o0[:, :64], torch.zeros_like(o0[:, :64])) and torch.equal(lse0[:, :64], torch.zeros_like(lse0[:, :64]))


def test_oracle_regression_pin(golden_dir):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(golden_dir, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    z = np.load(os.path.join(golden_dir, "oracle_config0.npz"))
    q, k, v, g, beta = mg.config0_inputs()
    types = otab.synth_types(2, 8, 4, 0.5, seed=0)
    assert np.array_equal(types.numpy(), z["types"])
    o_l, s_l = ogdn.linear_chunk(q, k, v, g, beta, types[..., 1], nbs=64)
    o_r, _ = ogdn.linear_recurrent(q, k, v, g, beta, types[..., 1], nbs=64)
    assert np.allclose(o_l[:, ::7].numpy(), z["o_lin"], atol=1e-5)
    assert (o_l - o_r).abs().max() < 1e-4        # fp32: chunk form vs naive recurrence
    mask = oattn.attn_mask(types[..., 0], 512, 64, 4)
    assert np.array_equal(mask.sum(-1).numpy().astype(np.int32), z["mask_rowsum"])
    o_a, lse = oattn.attn_sdpa(q, k, v, mask)
    assert np.allclose(o_a[:, ::7].numpy(), z["o_attn"], atol=1e-5)


def test_mamba_wrappers():
    B, T, H, K, V = 1, 256, 2, 16, 8
    q, k, v, g, _, h0 = _inputs(B, T, H, K, V, seed=5)
    ty = otab.synth_types(B, 1, 2, 0.1, seed=1)
    o1, s1 = omamba.mamba_recurrent(q, k, v, g, ty[..., 1], nbs=256, h0=h0)
    o2, s2 = omamba.mamba_chunk(q, k, v, g, ty[..., 1], nbs=256, h0=h0)
    assert (o1 - o2).abs().max() < 1e-11
