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


def _worker(rank, world, port, B, T, H, K, V, nbs, decay, seed, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from neuralattentionsearchlinear_b200.sequence_parallel import nats_mixed_attn_mamba_sp
        from tests.sp_helpers import OracleSegmentOps
        q, k, v, g, types = _inputs(B, T, H, K, V, nbs, seed)
        TN = types.shape[1]
        per = -(-TN // world)                      # blocks per rank (the last rank takes the rest, maybe ragged)
        b0, b1 = rank * per, min(TN, (rank + 1) * per)
        sl = slice(b0 * nbs, min(T, b1 * nbs))
        o_l, o_a, ht = nats_mixed_attn_mamba_sp(q[:, sl], k[:, sl], v[:, sl], q[:, sl], k[:, sl], v[:, sl], g[:, sl],
                                                types[:, b0:b1].contiguous(), nats_block_size=nbs,
                                                decay_for_non_mamba_blocks=decay, backend=OracleSegmentOps())
        ret[rank] = (o_l, o_a, ht)
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
    o_l = torch.cat([ret[r][0] for r in range(world)], 1)
    o_a = torch.cat([ret[r][1] for r in range(world)], 1)
    assert (o_l - o_ref).abs().max() < 1e-9
    assert (o_a - oa_ref).abs().max() < 1e-9
    # the final state is defined when the last block is selected (the layers force it)
    assert ret[world - 1][2] is not None and all(ret[r][2] is None for r in range(world - 1))
    assert (ret[world - 1][2] - s_ref).abs().max() < 1e-9


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
