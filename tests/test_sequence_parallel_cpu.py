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


def _worker(rank, world, port, B, T, H, K, V, nbs, decay, seed, ret, layout="contiguous", splits=None):
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
                                                linear_splits=splits, backend=OracleSegmentOps())
        ret[rank] = (o_l, o_a, ht, tsel)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,T,nbs,decay,splits", [(2, 1024, 128, True, None), (3, 1100, 128, True, None),
                                                      (2, 768, 256, False, None), (2, 1024, 128, True, 2),
                                                      (2, 1024, 256, False, 2)])
def test_sp_matches_single_process_oracle(world, T, nbs, decay, splits):
    B, H, K, V, seed = 1, 2, 16, 8, 3
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), B, T, H, K, V, nbs, decay, seed, ret, "contiguous", splits), nprocs=world,
             join=True)
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


@pytest.mark.parametrize("world,T,nbs,splits", [(2, 1024, 128, None), (3, 1536, 128, 2), (2, 2048, 128, 4)])
def test_sp_zigzag_matches_single_process_oracle(world, T, nbs, splits):
    B, H, K, V, seed = 2, 2, 16, 8, 5
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), B, T, H, K, V, nbs, True, seed, ret, "zigzag", splits), nprocs=world,
             join=True)
    q, k, v, g, types = _inputs(B, T, H, K, V, nbs, seed)
    o_ref, s_ref = ogdn.linear_recurrent(q, k, v, g, None, types[..., 1], nbs=nbs, scale=1.0, decay=True,
                                         use_l2norm=False, rule="mamba")
    mask = oattn.attn_mask(types[..., 0], T, nbs, H)
    oa_ref, _ = oattn.attn_sdpa(q, k, v, mask)
    _check(ret, world, o_ref, oa_ref, s_ref, holder=0)          # rank 0 holds segments 0 and 2*world-1


def test_virtual_types_layout():
    from neuralattentionsearchlinear_b200.sequence_parallel import virtual_attn_types
    n_all = torch.tensor([[[2, 0]], [[1, 3]], [[0, 1]]])          # [G=3, B=1, HN=2]
    local = torch.zeros(1, 2, 2, 2)
    local[0, 1, :, 0] = 1
    t = virtual_attn_types(n_all, torch.tensor([0, 1, 2]), [2], cap=3, types_local=local)
    assert t.shape == (1, 3 * 3 + 2, 2, 2)
    assert t[0, :, 0, 0].tolist() == [1, 1, 0, 1, 0, 0, 0, 0, 0, 0, 1]
    assert t[0, :, 1, 0].tolist() == [0, 0, 0, 1, 1, 1, 0, 0, 0, 0, 1]
    assert float(t[..., 1].abs().sum()) == 0.0
    # two local segments (global ids 1 and 2) over gathered segments in the order (0, 2, 1): segment-major batch
    local2 = torch.zeros(2, 2, 2, 2)
    t2 = virtual_attn_types(n_all, torch.tensor([0, 2, 1]), [1, 2], cap=3, types_local=local2)
    assert t2.shape == (2, 11, 2, 2)
    assert t2[0, :, 0, 0].tolist() == [1, 1, 0] + [0] * 8                  # segment 1 sees only segment 0
    assert t2[1, :, 0, 0].tolist() == [1, 1, 0, 0, 0, 0, 0, 0, 0, 0, 0]     # segment 2 sees 0 and 1 (gathered slot 2: n=0)
    assert t2[1, :, 1, 0].tolist() == [0, 0, 0, 0, 0, 0, 1, 0, 0, 0, 0]


def test_pick_linear_splits():
    from neuralattentionsearchlinear_b200.sequence_parallel import pick_linear_splits
    assert pick_linear_splits(65536, 256) == 64
    assert pick_linear_splits(4096, 256) == 4
    assert pick_linear_splits(1100, 128) == 1            # ragged
    assert pick_linear_splits(768, 256) == 1
    assert pick_linear_splits(2048, 64, target_tokens=512) == 4


def test_single_rank_sub_segment_split_matches_oracle():
    """One process, no process group: only the sub-segment split of the linear branch is exercised."""
    from neuralattentionsearchlinear_b200.sequence_parallel import nats_mixed_attn_mamba_sp
    from tests.sp_helpers import OracleSegmentOps
    B, T, H, K, V, nbs, seed = 2, 1024, 2, 16, 8, 128, 11
    q, k, v, g, types = _inputs(B, T, H, K, V, nbs, seed)
    types[:, -1] = 1
    for decay in (True, False):
        o_l, o_a, ht = nats_mixed_attn_mamba_sp(q, k, v, q, k, v, g, types, nats_block_size=nbs,
                                                decay_for_non_mamba_blocks=decay, linear_splits=4,
                                                backend=OracleSegmentOps())
        o_ref, s_ref = ogdn.linear_recurrent(q, k, v, g, None, types[..., 1], nbs=nbs, scale=1.0, decay=decay,
                                             use_l2norm=False, rule="mamba")
        oa_ref, _ = oattn.attn_sdpa(q, k, v, oattn.attn_mask(types[..., 0], T, nbs, H))
        assert (o_l - o_ref).abs().max() < 1e-9
        assert (o_a - oa_ref).abs().max() < 1e-9
        assert (ht - s_ref).abs().max() < 1e-9


# ------------------------------------------------------------------------------- failure on one rank (host side)
class _FailingOps:
    """Wraps the per-rank compute; on ``bad_rank`` the linear branch raises (or stalls for ``delay`` seconds) right before
    the (a, S) exchange, after the rank has already taken part in the first collective."""

    def __init__(self, inner, rank, bad_rank, delay):
        self._inner, self._rank, self._bad, self._delay = inner, rank, bad_rank, delay

    def __getattr__(self, name):
        return getattr(self._inner, name)

    def segment_decay(self, gcs, tables, decay):
        if self._rank == self._bad:
            if self._delay is None:
                raise RuntimeError("injected failure before the state exchange")
            import time
            time.sleep(self._delay)
        return self._inner.segment_decay(gcs, tables, decay)


def _failing_worker(rank, world, port, delay, ret):
    import datetime
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    try:
        from neuralattentionsearchlinear_b200.sequence_parallel import nats_mixed_attn_mamba_sp
        from tests.sp_helpers import OracleSegmentOps
        B, T, H, K, V, nbs = 1, 512, 2, 16, 16, 64
        q, k, v, g, types = _inputs(B, T, H, K, V, nbs, 5)
        per = T // world
        c = lambda x: x[:, rank * per:(rank + 1) * per].contiguous()
        ty = types[:, rank * (per // nbs):(rank + 1) * (per // nbs)].contiguous()
        ops = _FailingOps(OracleSegmentOps(), rank, bad_rank=1, delay=delay)
        try:
            o_l, o_a, _ = nats_mixed_attn_mamba_sp(c(q), c(k), c(v), c(q), c(k), c(v), c(g), ty, nats_block_size=nbs,
                                                   decay_for_non_mamba_blocks=True, backend=ops)
            ret[rank] = ("ok", bool(torch.isfinite(o_l).all() and torch.isfinite(o_a).all()))
        except Exception as e:                       # noqa: BLE001 - the test inspects whatever surfaced
            ret[rank] = ("error", f"{type(e).__name__}: {e}")
    finally:
        try:
            dist.destroy_process_group()
        except Exception:                            # noqa: BLE001
            pass


def _run_failing(delay):
    import time
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    t0 = time.time()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, delay, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    alive = [p.is_alive() for p in procs]
    for p in procs:
        if p.is_alive():
            p.kill()
    return dict(ret), alive, time.time() - t0


def test_rank_that_fails_before_the_state_exchange_surfaces_an_error():
    """Rank 1 raises on the host between two collectives and never sends its (a, S) pair: rank 0's exchange ends with
    an error (connection closed / process-group timeout) instead of blocking."""
    ret, alive, dt = _run_failing(delay=None)
    assert not any(alive), "a rank was still blocked after two minutes"
    assert ret[1][0] == "error" and "injected failure" in ret[1][1]
    assert ret[0][0] == "error", f"rank 0 should have seen the exchange fail, got {ret[0]}"
    assert dt < 100


def test_rank_that_is_late_for_the_state_exchange_is_waited_for():
    """Rank 1 sends its (a, S) pair three seconds late (inside the process-group timeout): the step completes."""
    ret, alive, dt = _run_failing(delay=3.0)
    assert not any(alive)
    assert ret[0] == ("ok", True) and ret[1] == ("ok", True)
