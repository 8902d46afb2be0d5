"""natsl_gdn_fwd_noalloc — the entry point for hosts that may not allocate device memory (a fixed
memory plan, a callback inside another runtime) — called through the C ABI and compared with the
regular entry points, which take their intermediates from caller-allocated buffers.

Two calls in a row with different inputs and shapes: the built-in scratch array is shared and keeps
the previous call's contents, so the second call would expose any stale read.  Collected last on
purpose (file name), and self-contained so that it also passes alone in a fresh process."""
import pytest
import torch

from oracle import tables as otab
from tests.helpers import assert_close, synth_gdn_inputs

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _run_both(nat, B, T, H, HN, K, V, nbs, seed, use_h0, warmed=False):
    from neuralattentionsearchlinear_b200 import _lib, _ops
    dev = torch.device("cuda", 0)
    q, k, v, g, beta, h0 = synth_gdn_inputs(B, T, H, K, V, seed=seed, normalize_qk=False)
    q, k, v, g, beta = (x.to(dev) for x in (q, k, v, g, beta))
    h0 = h0.to(dev) if use_h0 else None
    types = otab.synth_types(B, -(-T // nbs), HN, 0.35, seed=seed + 1).to(dev)
    tb = nat.build_selection_tables(types, T, nbs)
    scale = K ** -0.5
    # regular entry points (caller-provided intermediates)
    o_ref, ht_ref, _ = _ops.linear_fwd(_lib.RULE_GDN, q, k, v, g, beta, tb, scale, h0, True, True, True)
    # the no-allocation entry point: inputs and outputs only
    o = torch.empty(B, T, H, V, dtype=torch.bfloat16, device=dev)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    free_before = torch.cuda.mem_get_info(dev)[0]      # sees a raw cudaMalloc inside the library too
    _lib.call("natsl_gdn_fwd_noalloc", q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
              _lib.DT_BF16, tb.types_i.data_ptr(), tb.indices.data_ptr(), tb.n_blocks.data_ptr(), _lib.ptr(h0),
              o.data_ptr(), ht.data_ptr(), B, T, H, HN, K, V, nbs, scale, _lib.FLAG_DECAY_SKIPPED, 1,
              torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    if warmed:
        # the first call on a device may make the driver load the library's kernels; from the second call on the
        # device's free memory must not move (the intermediates of this shape would take about 6 MiB)
        assert abs(torch.cuda.mem_get_info(dev)[0] - free_before) < (1 << 20)
    assert_close(o, o_ref, TOL, "o (no-alloc vs regular)")
    assert_close(ht, ht_ref, TOL, "final state (no-alloc vs regular)")


def test_no_alloc_entry_matches_regular_path_twice():
    import neuralattentionsearchlinear_b200 as nat
    assert torch.cuda.is_available()
    _run_both(nat, 2, 700, 4, 2, 128, 128, 64, seed=3, use_h0=True)       # ragged last chunk, ~6 MB of scratch
    _run_both(nat, 1, 1024, 2, 2, 64, 128, 128, seed=4, use_h0=False)     # second call: other shape, stale scratch
    _run_both(nat, 2, 700, 4, 2, 128, 128, 64, seed=5, use_h0=True, warmed=True)   # kernels loaded: free memory fixed


def test_no_alloc_entry_rejects_before_launching():
    """A call the stages would refuse (here: value dim 96) is refused before anything is launched, so the output
    buffer keeps its contents."""
    from neuralattentionsearchlinear_b200 import _lib
    x = torch.zeros(4096, device="cuda")
    o = torch.full((4096,), 7.0, device="cuda")
    with pytest.raises(_lib.NatslError, match="unsupported head dims"):
        _lib.call("natsl_gdn_fwd_noalloc", *([x.data_ptr()] * 5), _lib.DT_BF16, *([x.data_ptr()] * 3), None,
                  o.data_ptr(), None, 1, 64, 1, 1, 64, 96, 64, 1.0, 0, 1, None)
    torch.cuda.synchronize()
    assert bool((o == 7.0).all())


def test_no_alloc_entry_rejects_oversize():
    from neuralattentionsearchlinear_b200 import _lib
    x = torch.zeros(1, device="cuda")
    with pytest.raises(_lib.NatslError, match="scratch holds"):
        _lib.call("natsl_gdn_fwd_noalloc", *([x.data_ptr()] * 5), _lib.DT_BF16, *([x.data_ptr()] * 3), None,
                  x.data_ptr(), None, 8, 4096, 16, 16, 128, 128, 64, 1.0, 0, 1, None)
