"""Sequence-parallel host logic with gloo ranks on CPU: the per-rank compute is the oracle (tests/sp_helpers.py),
the exchange, state fold and virtual key sequence are the package's own code; the result must equal the
single-process oracle on the whole sequence."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attn as oattn
from oracle import gdn as ogdn
from oracle import tables as otab


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(B, T, H, K, V, nbs, seed):
    g_ = torch.Generator().manual_seed(seed)
    dt = torch.float64
    q = torch.randn(B, T, H, K, generator=g_, dtype=dt) * K ** -0.25
    k = torch.randn(B, T, H, K, generator=g_, dtype=dt) * K ** -0.25
    v = torch.randn(B, T, H, V, generator=g_, dtype=dt)
    g = -torch.nn.functional.softplus(torch.randn(B, T, H, generator=g_, dtype=dt) - 1.0) * 0.1
    types = otab.synth_types(B, -(-T // nbs), H, 0.3, seed=seed + 1, dtype=dt)
    return q, k, v, g, types


def _worker(rank, world, port, B, T, H, K, V, nbs, decay, seed, ret, layout="contiguous"):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from neuralattentionsearchlinear_b200.sequence_parallel import nats_mixed_attn_mamba_sp
        from tests.sp_helpers import OracleSegmentOps
        q, k, v, g, types = _inputs(B, T, H, K, V, nbs, seed)
        TN = types.shape[1]
        if layout == "contiguous":
            per = -(-TN // world)                  # blocks per rank (the last rank takes the rest, maybe ragged)
            b0, b1 = rank * per, min(TN, (rank + 1) * per)
            tsel = torch.arange(b0 * nbs, min(T, b1 * nbs))
            bsel = torch.arange(b0, b1)
        else:
            from neuralattentionsearchlinear_b200.sequence_parallel import segment_ids
            per = TN // (2 * world)                # blocks per segment
            ids = segment_ids(rank, world, "zigzag")
            tsel = torch.cat([torch.arange(s * per * nbs, (s + 1) * per * nbs) for s in ids])
            bsel = torch.cat([torch.arange(s * per, (s + 1) * per) for s in ids])
        c = lambda x: x[:, tsel].contiguous()
        o_l, o_a, ht = nats_mixed_attn_mamba_sp(c(q), c(k), c(v), c(q), c(k), c(v), c(g), types[:, bsel].contiguous(),
                                                nats_block_size=nbs, decay_for_non_mamba_blocks=decay, layout=layout,
                                                backend=OracleSegmentOps())
        ret[rank] = (o_l, o_a, ht, tsel)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,T,nbs,decay", [(2, 1024, 128, True), (3, 1100, 128, True), (2, 768, 256, False)])
def test_sp_matches_single_process_oracle(world, T, nbs, decay):
    B, H, K, V, seed = 1, 2, 16, 8, 3
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), B, T, H, K, V, nbs, decay, seed, ret), nprocs=world, join=True)
    q, k, v, g, types = _inputs(B, T, H, K, V, nbs, seed)
    o_ref, s_ref = ogdn.linear_recurrent(q, k, v, g, None, types[..., 1], nbs=nbs, scale=1.0, decay=decay,
                                         use_l2norm=False, rule="mamba")
    mask = oattn.attn_mask(types[..., 0], T, nbs, H)
    oa_ref, _ = oattn.attn_sdpa(q, k, v, mask)
    _check(ret, world, o_ref, oa_ref, s_ref, holder=world - 1)


def _check(ret, world, o_ref, oa_ref, s_ref, holder):
    for r in range(world):
        o_l, o_a, ht, tsel = ret[r]
        assert (o_l - o_ref[:, tsel]).abs().max() < 1e-9
        assert (o_a - oa_ref[:, tsel]).abs().max() < 1e-9
        # the final state is defined when the last block is selected (the layers force it)
        assert (ht is not None) == (r == holder)
    assert (ret[holder][2] - s_ref).abs().max() < 1e-9


@pytest.mark.parametrize("world,T,nbs", [(2, 1024, 128), (3, 1536, 128)])
def test_sp_zigzag_matches_single_process_oracle(world, T, nbs):
    B, H, K, V, seed = 2, 2, 16, 8, 5
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), B, T, H, K, V, nbs, True, seed, ret, "zigzag"), nprocs=world, join=True)
    q, k, v, g, types = _inputs(B, T, H, K, V, nbs, seed)
    o_ref, s_ref = ogdn.linear_recurrent(q, k, v, g, None, types[..., 1], nbs=nbs, scale=1.0, decay=True,
                                         use_l2norm=False, rule="mamba")
    mask = oattn.attn_mask(types[..., 0], T, nbs, H)
    oa_ref, _ = oattn.attn_sdpa(q, k, v, mask)
    _check(ret, world, o_ref, oa_ref, s_ref, holder=0)          # rank 0 holds segments 0 and 2*world-1


def test_virtual_types_layout():
    from neuralattentionsearchlinear_b200.sequence_parallel import virtual_attn_types
    n_all = torch.tensor([[[2, 0]], [[1, 3]], [[0, 1]]])          # [world=3, B=1, HN=2]
    local = torch.zeros(1, 2, 2, 2)
    local[0, 1, :, 0] = 1
    t = virtual_attn_types(n_all, rank=2, cap=3, types_local=local)
    assert t.shape == (1, 3 * 3 + 2, 2, 2)
    assert t[0, :, 0, 0].tolist() == [1, 1, 0, 1, 0, 0, 0, 0, 0, 0, 1]
    assert t[0, :, 1, 0].tolist() == [0, 0, 0, 1, 1, 1, 0, 0, 0, 0, 1]
    assert float(t[..., 1].abs().sum()) == 0.0
