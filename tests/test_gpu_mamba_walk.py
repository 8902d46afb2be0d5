"""GPU tests (-m gpu) of the fused Mamba2 walk (`natsl_mamba_walk_fused`, tcgen05: recurrence + chunk output with the state
in tensor memory) against the oracle's chunk form (src/nats/ops/mamba/chunk_h.py:139-218, chunk_o.py:137-198) and against
the two-kernel path it replaces (`natsl_linear_fwd_h` + `natsl_linear_fwd_o`)."""
import pytest
import torch

from oracle import gdn as ogdn
from oracle import tables as otab
from tests.helpers import assert_close, synth_mamba_inputs

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def nat():
    import neuralattentionsearchlinear_b200 as nat
    return nat


def _both(nat, q, k, v, g, h0, types, T, nbs, decay, skip_out=False, quirk=True):
    """-> (fused walk result, two-kernel result), each (o, ht)."""
    from neuralattentionsearchlinear_b200 import _lib, _ops
    tb = nat.build_selection_tables(types.cuda(), T, nbs)
    cu = lambda x: None if x is None else x.cuda()
    out = []
    for fused in (True, False):
        old = _ops.USE_MAMBA_WALK
        _ops.USE_MAMBA_WALK = fused
        try:
            o, ht, _ = _ops.linear_fwd(_lib.RULE_MAMBA, cu(q), cu(k), cu(v), cu(g), None, tb, 1.0, cu(h0), decay, False, True,
                                       trailing_quirk=quirk, skip_out=skip_out)
        finally:
            _ops.USE_MAMBA_WALK = old
        torch.cuda.synchronize()
        assert _lib.load().natsl_device_status() == 0
        out.append((o, ht))
    return out


@pytest.mark.parametrize("B,T,H,HN,nbs,decay,p_lin,with_h0", [
    (1, 1024, 4, 4, 256, True, 0.8, True),       # the long-context configuration's block size
    (2, 512, 2, 2, 64, True, 0.5, False),        # chunk == block: unselected chunks only carry the decay
    (1, 900, 2, 1, 128, False, 0.5, True),       # ragged last chunk, one selection head for two heads, no carried decay
    (1, 700, 3, 3, 256, True, 0.3, False),       # ragged last block that is mostly unselected
    (2, 256, 2, 2, 64, True, 0.0, True),         # nothing selected: the state never changes
    (1, 640, 2, 2, 128, True, 1.0, False),       # everything selected
])
def test_walk_matches_the_oracle_and_the_two_kernel_path(nat, B, T, H, HN, nbs, decay, p_lin, with_h0):
    K, V = 128, 64
    q, k, v, g, h0 = synth_mamba_inputs(B, T, H, K, V, seed=T + nbs)
    if not with_h0:
        h0 = None
    types = otab.synth_types(B, -(-T // nbs), HN, 1.0 - p_lin, seed=T + 1)
    (o, ht), (o2, ht2) = _both(nat, q, k, v, g, h0, types, T, nbs, decay)
    o_ref, s_ref = ogdn.linear_chunk(q.float(), k.float(), v.float(), g, None, types[..., 1], nbs=nbs, scale=1.0, h0=h0,
                                     decay=decay, use_l2norm=False, rule="mamba")
    assert_close(o, o_ref, TOL, "o (fused walk)")
    assert_close(ht, s_ref, 2 * TOL, "final state (fused walk)")
    assert_close(o, o2, TOL, "o: fused walk vs scan + out")
    assert_close(ht, ht2, 2 * TOL, "final state: fused walk vs scan + out")


def test_walk_state_only_and_reproducible(nat):
    """Without an output the walk returns the same final state; two runs are bit-identical."""
    B, T, H, K, V, nbs = 2, 1024, 4, 128, 64, 256
    q, k, v, g, h0 = synth_mamba_inputs(B, T, H, K, V, seed=3)
    types = otab.synth_types(B, T // nbs, H, 0.4, seed=4)
    (o, ht), _ = _both(nat, q, k, v, g, h0, types, T, nbs, True)
    (o_b, ht_b), _ = _both(nat, q, k, v, g, h0, types, T, nbs, True)
    assert torch.equal(o, o_b) and torch.equal(ht, ht_b)
    (o_s, ht_s), (_, ht_s2) = _both(nat, q, k, v, g, h0, types, T, nbs, True, skip_out=True)
    assert o_s is None
    assert torch.equal(ht_s, ht)
    assert_close(ht_s, ht_s2, 2 * TOL, "state-only: fused walk vs scan")


def test_walk_without_the_trailing_quirk(nat):
    B, T, H, K, V, nbs = 1, 768, 2, 128, 64, 64
    q, k, v, g, h0 = synth_mamba_inputs(B, T, H, K, V, seed=9)
    types = otab.synth_types(B, T // nbs, H, 0.6, seed=10)
    (o, ht), (o2, ht2) = _both(nat, q, k, v, g, h0, types, T, nbs, True, quirk=False)
    assert_close(o, o2, TOL, "o: fused walk vs scan + out (no trailing quirk)")
    assert_close(ht, ht2, 2 * TOL, "final state (no trailing quirk)")


def test_walk_refuses_other_head_dims():
    from neuralattentionsearchlinear_b200 import _lib
    z = torch.zeros(1, 64, 1, 128, dtype=torch.bfloat16, device="cuda")
    f = torch.zeros(1, 64, 1, dtype=torch.float32, device="cuda")
    i = torch.zeros(1, 1, 1, 2, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.NatslError):
        _lib.call("natsl_mamba_walk_fused", z.data_ptr(), z.data_ptr(), z.data_ptr(), f.data_ptr(), i.data_ptr(), i.data_ptr(),
                  i.data_ptr(), None, z.data_ptr(), None, 1, 64, 1, 1, 128, 128, 64, 1.0, 0, None)
