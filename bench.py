#!/usr/bin/env python
"""Benchmark of the NAtSL-GDN hybrid attention layer forward (prefill) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one call of ``nats_mixed_attn_gdn`` (selection tables, chunk-masked softmax branch,
gated-delta-rule branch) on one batch of seeded synthetic tensors of the single-GPU layer
configuration: B=8, T=4096, H=HQ=16, d_k=d_v=128, block 64, bf16 in / fp32 accumulate, about
25 % of (block, head) pairs softmax-selected, last block forced, decay over skipped blocks on.
With N GPUs every rank runs its own batch (independent (batch, head) units, no collective in the
data path: weak scaling); the timed region is bracketed by a barrier and a device synchronise and
the time is the maximum over ranks.  Prints ONE JSON line on rank 0.

``--workload mamba_long`` (optional) runs the long-context NAtSL-Mamba2 layer (B=1, T=65536, H=32, block 256),
sequence-parallel over the ranks (strong scaling); ``--sp-plan`` uses the plan / replay form.

``--impl reference`` times the reference algorithm's CPU form (the PyTorch restatement under
``oracle/``; the reference's own code is Triton-only and cannot run on host cores) on a bounded
sample of the same workload, on rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=8, T=4096, H=16, K=128, V=128, nbs=64, p_attn=0.25)
WORKLOAD = "natsl_gdn_layer_fwd B={B} T=4096 H=HQ=16 dk=dv=128 block=64 bf16 p_softmax=0.25"


def layer_config(world: int, B: int) -> dict:
    """The ``config`` object of the JSON line: the same for both arms (the reference arm times the same workload)."""
    return {"workload": WORKLOAD.format(B=B), "per_gpu_batch": B,
            "parallelism": f"replicas x{world} (batch sharded, no collective)",
            "l2": "inputs and intermediates (>0.9 GB per step) exceed the 126 MB L2; no explicit flush"}


def init_process_group_quiet(dev):
    """NCCL process group; whatever the libraries print while the communicator comes up (NCCL's version banner) goes
    to stderr, so that stdout carries the one JSON line only."""
    import torch.distributed as dist
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
        torch.cuda.synchronize(dev)
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)
    return dist


# ------------------------------------------------------------------------------- inputs
def make_inputs(seed: int, B: int, H: int):
    """Host tensors (fp32 generation on CPU, cast to bf16).  q, k L2-normalised per head."""
    T, K, V, nbs = CFG["T"], CFG["K"], CFG["V"], CFG["nbs"]
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=gen)
    k = torch.randn(B, T, H, K, generator=gen)
    v = torch.randn(B, T, H, V, generator=gen)
    q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6)
    k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.randn(B, T, H, generator=gen).sigmoid()
    g = -torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen))
    # selection: logits ~ N(0,1), attention logit shifted so that P(softmax) = p_attn; hard argmax; last block forced
    TN = T // nbs
    logits = torch.randn(B, TN, H, 2, generator=gen)
    shift = (2.0 ** 0.5) * torch.distributions.Normal(0.0, 1.0).icdf(torch.tensor(CFG["p_attn"])).item()
    logits[..., 0] += shift
    types = torch.zeros_like(logits).scatter_(-1, logits.softmax(-1).max(-1, keepdim=True)[1], 1.0)
    types[:, -1] = 1
    return dict(q=q.bfloat16(), k=k.bfloat16(), v=v.bfloat16(), g=g, beta=beta.bfloat16(), types=types.bfloat16())


def attention_tile_flops(types: torch.Tensor, H: int, DK: int, DV: int, C: int = 64) -> float:
    """Algorithmic FLOPs of the softmax branch: 2*(DK+DV)*C^2 per visible (query chunk, key chunk)
    pair = own chunk + every softmax-selected earlier chunk."""
    sel = types[..., 0].float()                                   # [B,TN,HN]
    B, TN, HN = sel.shape
    later = torch.arange(TN - 1, -1, -1, dtype=torch.float32).view(1, TN, 1)   # chunks after c
    pairs = (sel * later).sum() * (H // HN) + B * H * TN
    return float(pairs) * 2.0 * (DK + DV) * C * C


# ------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if val == "Active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------- CPU arms
def cpu_oracle_step(inp, b_slice: int, h_slice: int):
    """Reference algorithm (chunk form + masked SDPA) on CPU for a [b_slice, :, h_slice] sample."""
    from oracle import attn as oattn
    from oracle import gdn as ogdn
    sl = lambda x: x[:b_slice, :, :h_slice].float().contiguous()
    q, k, v, g, beta = (sl(inp[n]) for n in ("q", "k", "v", "g", "beta"))
    types = inp["types"][:b_slice, :, :h_slice].float()
    T, nbs = CFG["T"], CFG["nbs"]
    o_l, _ = ogdn.linear_chunk(q, k, v, g, beta, types[..., 1], nbs=nbs, decay=True)
    mask = oattn.attn_mask(types[..., 0], T, nbs, h_slice)
    o_a, _ = oattn.attn_sdpa(q, k, v, mask)
    return o_l, o_a


def time_cpu_baseline(inp, budget_s: float, reps: int = 1):
    """Times the oracle on a bounded sample sized to roughly `budget_s` seconds per repetition."""
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    cpu_oracle_step(inp, 1, 1)
    unit = time.perf_counter() - t0                       # one (batch, head) unit
    H = CFG["H"]
    hs = max(1, min(H, int(budget_s / max(unit, 1e-3))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        outs = cpu_oracle_step(inp, 1, hs)
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    tokens = CFG["T"] * hs / H                            # token-equivalents of the full-head layer
    return tokens / dt, f"1 of 8 sequences x {hs} of {H} heads, T=4096 (linear in heads and batch)", dt, outs, hs


def run_reference(args, rank: int):
    if rank != 0:
        return
    inp = make_inputs(0, 1, CFG["H"])
    total = max(1, args.steps + args.warmup)
    per_step = min(20.0, 150.0 / total)
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    cpu_oracle_step(inp, 1, 1)
    unit = time.perf_counter() - t0
    hs = max(1, min(CFG["H"], int(per_step / max(unit, 1e-3))))
    for _ in range(args.warmup):
        cpu_oracle_step(inp, 1, hs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_oracle_step(inp, 1, hs)
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    val = CFG["T"] * hs / CFG["H"] / dt
    sample = f"per step: 1 of 8 sequences x {hs} of {CFG['H']} heads, T=4096"
    cores = torch.get_num_threads()
    print(json.dumps({
        "impl": "reference", "metric": "prefill_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
        "config": layer_config(args.gpus, CFG["B"]),
        "note": "reference algorithm restated in PyTorch on host cores (the reference's own implementation is Triton-only)",
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------- GPU arm
def run_ours(args, rank: int, world: int, local_rank: int):
    import neuralattentionsearchlinear_b200 as nat
    from neuralattentionsearchlinear_b200 import _lib, _ops
    _lib.load()                                           # fail loudly if the CUDA library is missing
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU fallback for the hot path")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        dist = init_process_group_quiet(dev)
    B, T, H, K, V, nbs = (CFG[n] for n in ("B", "T", "H", "K", "V", "nbs"))
    host = make_inputs(1000 * rank, B, H)
    pinned = {n: t.pin_memory() for n, t in host.items()}
    d = {n: t.to(dev) for n, t in host.items()}
    stream = torch.cuda.current_stream(dev)

    def step(x):
        return nat.nats_mixed_attn_gdn(x["q"], x["k"], x["v"], x["q"], x["k"], x["v"], None, x["g"], x["beta"],
                                       x["types"], None, nats_block_size=nbs, ops_for_incomplete_chunks="all",
                                       output_final_state_gated_delta=True, decay_for_non_gdn_blocks=True)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up: at least W steps and at least ~1.5 s of load, so that clocks settle and the clock
    # sampler (started first) has samples under the same load as the timed region that follows directly
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    clocks = ClockSampler(vis.split(",")[local_rank].strip() if vis else local_rank)
    if rank == 0:
        clocks.start()
    n_warm = max(3, args.warmup)
    for _ in range(n_warm):
        out = step(d)
    torch.cuda.synchronize(dev)
    t_w = time.perf_counter()
    while time.perf_counter() - t_w < args.min_warm_seconds:
        for _ in range(20):
            out = step(d)
        torch.cuda.synchronize(dev)
    if rank == 0:
        clocks.rows.clear()          # keep only samples taken under load
    # ---- device-resident throughput.  The step (tables, both branches on their two streams) is captured once into a
    # CUDA graph and replayed: the timed region then holds device work only, whatever the host does meanwhile (issuing
    # the step eagerly takes about as long on the host as it runs on the device, so a busy host shows up in the number).
    # The eager figure is reported beside it.
    graph, launches_per_step = None, None
    if not args.no_graph:
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                g_ = torch.cuda.CUDAGraph()
                n0 = _lib.kernel_launches()
                # thread-local error mode: calls made by other threads (NCCL's watchdog) do not break the capture
                with torch.cuda.graph(g_, stream=side, capture_error_mode="thread_local"):
                    g_out = step(d)
                launches_per_step = _lib.kernel_launches() - n0
            stream.wait_stream(side)
            torch.cuda.synchronize(dev)
            g_.replay()
            torch.cuda.synchronize(dev)
            ref_out = step(d)
            torch.cuda.synchronize(dev)
            if all(torch.equal(a, b) for a, b in zip(g_out, ref_out)):
                graph = g_
        except Exception as exc:                            # capture is an optimisation of the measurement, not a need
            print(f"[bench] CUDA graph capture of the step failed ({type(exc).__name__}: {exc}); timing eagerly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize(dev)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = _lib.kernel_launches()
    e0.record(stream)
    for _ in range(args.steps):
        out = step(d)
    e1.record(stream)
    gpu_launches = _lib.kernel_launches() - launches_before      # kernels of this library launched in the timed region
    barrier()
    ms_eager = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    ms_total = ms_eager * args.steps
    if graph is not None:
        for _ in range(3):
            graph.replay()
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        barrier()
        ms_total = max_over_ranks(e0.elapsed_time(e1))
        gpu_launches = launches_per_step * args.steps
        out = g_out
    if rank == 0 and len(clocks.rows) < 3 and args.min_warm_seconds > 0:
        # the timed region was shorter than the sampling period: keep the same load up until a few samples exist
        t_w = time.perf_counter()
        while len(clocks.rows) < 3 and time.perf_counter() - t_w < 3.0:
            for _ in range(20):
                out = step(d)
            torch.cuda.synchronize(dev)
    clk = clocks.stop() if rank == 0 else None
    barrier()
    ms_step = ms_total / args.steps
    value = world * B * T / (ms_step * 1e-3)

    # ---- per-kernel durations: each stage launched `steps` times back to back on the same stream between two
    # CUDA events (the queue stays full, so the events bracket device time, not host launch latency)
    names = ["tables", "attn_fwd", "gdn_prep", "gdn_prep_mma_sync", "walk_fused", "walk_vsplit", "scan_fwd_h", "out_fwd_o"]
    NT = T // 64
    tb = nat.build_selection_tables(d["types"], T, nbs)
    gcs = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    krs = torch.empty_like(gcs)
    qrs = torch.empty_like(gcs)
    pmat = torch.empty(B, T, H, 64, dtype=torch.bfloat16, device=dev)
    w = torch.empty(B, T, H, K, dtype=torch.bfloat16, device=dev)
    u = torch.empty(B, T, H, V, dtype=torch.bfloat16, device=dev)
    hbuf = torch.empty(B, NT, H, K, V, dtype=torch.bfloat16, device=dev)
    carry = torch.empty(B, NT, H, dtype=torch.float32, device=dev)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=dev)
    o = torch.empty(B, T, H, V, dtype=torch.bfloat16, device=dev)
    sp = stream.cuda_stream
    stages = {
        "tables": lambda: nat.build_selection_tables(d["types"], T, nbs),
        "attn_fwd": lambda: _ops.attn_fwd(d["q"], d["k"], d["v"], tb, K ** -0.5, True),
        "gdn_prep": lambda: _lib.call(_ops.prep_entry(K, V), d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(),
                                      d["g"].data_ptr(), d["beta"].data_ptr(), _lib.DT_BF16, w.data_ptr(), u.data_ptr(),
                                      gcs.data_ptr(), krs.data_ptr(), qrs.data_ptr(), pmat.data_ptr(), B, T, H, K, V, 1, sp),
        "gdn_prep_mma_sync": lambda: _lib.call("natsl_gdn_chunk_prep_ex", d["q"].data_ptr(), d["k"].data_ptr(),
                                               d["v"].data_ptr(), d["g"].data_ptr(), d["beta"].data_ptr(), _lib.DT_BF16,
                                               w.data_ptr(), u.data_ptr(), gcs.data_ptr(), krs.data_ptr(), qrs.data_ptr(),
                                               pmat.data_ptr(), B, T, H, K, V, 1, sp),
        "walk_fused": lambda: _lib.call("natsl_gdn_walk_fused", d["q"].data_ptr(), d["k"].data_ptr(), w.data_ptr(),
                                        u.data_ptr(), pmat.data_ptr(), gcs.data_ptr(), krs.data_ptr(), qrs.data_ptr(),
                                        tb.types_i.data_ptr(), tb.indices.data_ptr(), tb.n_blocks.data_ptr(), None,
                                        o.data_ptr(), ht.data_ptr(), B, T, H, H, K, V, nbs, K ** -0.5,
                                        _lib.FLAG_DECAY_SKIPPED, sp),
        "walk_vsplit": lambda: _lib.call("natsl_gdn_walk_fused_vsplit", d["q"].data_ptr(), d["k"].data_ptr(), w.data_ptr(),
                                         u.data_ptr(), pmat.data_ptr(), gcs.data_ptr(), krs.data_ptr(), qrs.data_ptr(),
                                         tb.types_i.data_ptr(), tb.indices.data_ptr(), tb.n_blocks.data_ptr(), None,
                                         o.data_ptr(), ht.data_ptr(), B, T, H, H, K, V, nbs, K ** -0.5,
                                         _lib.FLAG_DECAY_SKIPPED, sp),
        "scan_fwd_h": lambda: _lib.call("natsl_linear_fwd_h", _lib.RULE_GDN, d["k"].data_ptr(), w.data_ptr(), u.data_ptr(),
                                        gcs.data_ptr(), krs.data_ptr(), tb.types_i.data_ptr(), tb.indices.data_ptr(),
                                        tb.n_blocks.data_ptr(), None, hbuf.data_ptr(), carry.data_ptr(), ht.data_ptr(),
                                        B, T, H, H, K, V, nbs, _lib.FLAG_DECAY_SKIPPED, sp),
        "out_fwd_o": lambda: _lib.call("natsl_linear_fwd_o", _lib.RULE_GDN, d["q"].data_ptr(), d["k"].data_ptr(),
                                       w.data_ptr(), u.data_ptr(), gcs.data_ptr(), krs.data_ptr(), hbuf.data_ptr(),
                                       carry.data_ptr(), o.data_ptr(), B, T, H, K, V, K ** -0.5, 1, sp),
    }
    kernel_ms = {}
    for n in names:                      # in pipeline order, so every stage sees valid inputs
        stages[n]()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            stages[n]()
        ev1.record(stream)
        torch.cuda.synchronize(dev)
        kernel_ms[n] = ev0.elapsed_time(ev1) / args.steps
    if _lib.load().natsl_device_status() != 0:
        raise RuntimeError("a kernel reported a failed bounded wait: " + _lib.load().natsl_last_error().decode())

    # ---- end to end: host (pinned) inputs -> device -> op -> host outputs, every step
    h2d = sum(t.numel() * t.element_size() for t in pinned.values())
    d2h = 2 * B * T * H * V * 2 + B * H * K * V * 4
    e2e_steps = args.steps

    # Every step copies its inputs from pinned host memory and its outputs back; the copies of neighbouring steps
    # overlap the compute (PCIe is full duplex): an upload stream, the compute stream and a download stream, two
    # sets of device input buffers and host output buffers.
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    x_dev = [{n: torch.empty_like(t, device=dev) for n, t in pinned.items()} for _ in range(2)]
    o_host = [[torch.empty(B, T, H, V, dtype=torch.bfloat16).pin_memory() for _ in range(2)] for _ in range(2)]
    ht_host = [torch.empty(B, H, K, V, dtype=torch.float32).pin_memory() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        b2 = i & 1
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_comp[b2])              # the step that last read this input set has finished
            for n, t in pinned.items():
                x_dev[b2][n].copy_(t, non_blocking=True)
            ev_in[b2].record(s_in)
        stream.wait_event(ev_in[b2])
        og, oa, hts = step(x_dev[b2])
        ev_comp[b2].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b2])
            o_host[b2][0].copy_(og, non_blocking=True)
            o_host[b2][1].copy_(oa, non_blocking=True)
            ht_host[b2].copy_(hts, non_blocking=True)
            ev_out[b2].record(s_out)
        for t_ in (og, oa, hts):
            t_.record_stream(s_out)

    def e2e_drain():
        stream.wait_stream(s_out)
        stream.wait_stream(s_in)

    for i in range(2):
        e2e_step(i)
    e2e_drain()
    barrier()
    e0.record(stream)
    for i in range(e2e_steps):
        e2e_step(i + 2)
    e2e_drain()
    e1.record(stream)
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    e2e_value = world * B * T / (e2e_ms * 1e-3)

    # ---- N > 1: the long-context layer split over the ranks (the configuration the multi-GPU target is about), and
    # the same layer on one GPU, measured in this run: every rank runs the one-GPU case side by side on its own GPU
    sp_info = None
    if dist is not None and not args.no_sp:
        lin_group = dist.new_group()
        solo = None
        for r in range(world):
            gr = dist.new_group([r])
            if r == rank:
                solo = gr
        r_n = mamba_long_measure(args, rank, world, dev, group=None, lin_group=lin_group, plan=True, parity=True)
        barrier()
        # the same layer on one GPU, in this run: rank 0 alone, the other ranks wait at the barrier (no host contention)
        r_1 = mamba_long_measure(args, 0, 1, dev, group=solo, lin_group=None, plan=False, parity=False) if rank == 0 else None
        barrier()
        if rank == 0:
            one = r_1["ms_per_step"]
            sp_info = {"workload": "natsl_mamba2_layer_fwd B=1 T=65536 H=32 dstate=128 dhead=64 block=256 p_softmax=0.10",
                       "scaling": "strong", "n_gpus": world, "ms_per_step": r_n["ms_per_step"],
                       "tokens_per_s": r_n["tokens_per_s"], "one_gpu_ms_per_step": one,
                       "one_gpu_host_issue_ms_per_step": r_1["host_issue_ms_per_step"],
                       "speedup_vs_one_gpu": one / r_n["ms_per_step"], "launch": r_n["launch"], "layout": r_n["layout"],
                       "host_issue_ms_per_step": r_n["host_issue_ms_per_step"], "parity": r_n.get("parity"),
                       "device_status": _lib.load().natsl_device_status()}
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    # ---- rooflines: algorithmic work of each stage / its measured time, against the measured peaks
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peaks = json.load(open(peaks_path))
        peak_tf, peak_bw = float(peaks["bf16_tflops_sustained"]), float(peaks["hbm_gbs"])
        peak_src = "measured (MEASURED_PEAKS.json: sustained bf16 GEMM / copy bandwidth)"
    else:
        peak_tf, peak_bw, peak_src = 1400.0, 6650.0, "fallback"
    n_tok = B * T * H
    frac_lin = float(host["types"][..., 1].float().mean())
    state_bytes = B * NT * H * K * V * 2
    # DRAM bytes per launch from a profiler capture at a smaller batch (tracked file; it names the build it was taken
    # from), scaled by the batch: traffic grows in proportion to the independent (batch, head) units
    traffic_path = os.path.join(ROOT, "profiles", "dram_traffic_per_launch.json")
    ncu_traffic, ncu_batch = {}, 1
    if os.path.exists(traffic_path):
        tr = json.load(open(traffic_path))
        ncu_traffic, ncu_batch = tr["bytes_per_launch"], tr["batch"]
    # the step runs tables, attn_fwd, gdn_prep, walk_fused; scan_fwd_h + out_fwd_o are the two-kernel path the fused
    # walk replaces at this shape (still used for other head dims / block sizes) and are timed for comparison
    walk_stage = "walk_vsplit" if _ops.WALK_VSPLIT else "walk_fused"
    in_step = ("attn_fwd", "gdn_prep", walk_stage)
    work = {
        # reads q, k, w, u, P once, writes o
        "walk_fused": ("hbm", n_tok * (3 * K + V + 64) * 2 + n_tok * V * 2, "gdn_walk_tc_kernel"),
        "walk_vsplit": ("hbm", n_tok * (3 * K + V + 64) * 2 + n_tok * V * 2, "gdn_walk_half_kernel"),
        "attn_fwd": ("tensor", attention_tile_flops(host["types"], H, K, V), "attn_fwd_tc_kernel<128,128>"),
        "gdn_prep": ("hbm", n_tok * (2 * K + V) * 2 + n_tok * (K + V + 64) * 2 + n_tok * 18,
                     "gdn_prep_tc_kernel" if _ops.prep_entry(K, V).endswith("_tc") else "gdn_prep_kernel<128,128>"),
        "gdn_prep_mma_sync": ("hbm", n_tok * (2 * K + V) * 2 + n_tok * (K + V + 64) * 2 + n_tok * 18, "gdn_prep_kernel<128,128>"),
        "scan_fwd_h": ("hbm", frac_lin * n_tok * (2 * K + V) * 2 + state_bytes, "linear_scan_kernel<128,32,gdn>"),
        "out_fwd_o": ("hbm", n_tok * (3 * K + V) * 2 + state_bytes + n_tok * V * 2, "linear_out_kernel<128,128,gdn>"),
    }
    roofs = {}
    for n, (bound, amount, kname) in work.items():
        sec = kernel_ms[n] * 1e-3
        if bound == "tensor":
            ach, peak, unit = amount / sec / 1e12, peak_tf, "TFLOP/s"
        else:
            ach, peak, unit = amount / sec / 1e9, peak_bw, "GB/s"
        roofs[n] = {"kernel": kname, "bound": bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                    "traffic": (ncu_traffic[n] * B / ncu_batch) if ncu_traffic.get(n) else None, "algorithmic_per_launch": amount,
                    "ms_per_launch": kernel_ms[n]}
    dom = max(in_step, key=lambda n: kernel_ms[n])
    roofline = dict(roofs[dom], peak_source=peak_src, dominant_stage=dom)
    # ---- CPU baseline (oracle port) on a bounded sample
    cpu_val, cpu_sample, _, (ref_l, ref_a), hs = time_cpu_baseline({n: t for n, t in host.items()}, budget_s=15.0)
    # output error of the timed device path against the oracle on the sample the oracle just computed
    err_l = float((out[0][:1, :, :hs].float().cpu() - ref_l).abs().max())
    err_a = float((out[1][:1, :, :hs].float().cpu() - ref_a).abs().max())
    mag = float(max(ref_l.abs().max(), ref_a.abs().max()))
    line = {
        "metric": "prefill_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded, generated on the host)",
        "config": layer_config(world, B),
        "clocks": clk, "gpu_launches": gpu_launches,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps,
                "pipelining": "uploads, compute and downloads of neighbouring steps overlap (three streams, two buffer sets)"},
        "launch": "one CUDA graph per step, replayed" if graph is not None else "eager", "ms_per_step_eager": ms_eager,
        "kernel_ms": kernel_ms, "roofline": roofline, "roofline_all": roofs,
        "cpu_baseline": {"value": cpu_val, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": cpu_sample},
        "sp_long_context": sp_info,
        "parity": {"max_abs_err_o_gdn": err_l, "max_abs_err_o_attn": err_a, "max_abs_ref": mag, "tolerance": "rtol=atol=1e-2",
                   "sample": f"sequence 0, heads 0..{hs - 1}, device outputs of the timed step vs the fp32 CPU oracle"},
    }
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------- long-context Mamba2 (optional)
MAMBA_LONG = dict(T=65536, H=32, K=128, V=64, nbs=256, p_attn=0.10)


def mamba_long_segment(sid: int, n_glob: int, L: int):
    """Host tensors of segment ``sid`` of the long-context input, generated from the segment's own seed."""
    c = MAMBA_LONG
    H, K, V, nbs = c["H"], c["K"], c["V"], c["nbs"]
    A = -torch.exp(torch.rand(H, generator=torch.Generator().manual_seed(4)) * torch.log(torch.tensor(16.0)))
    shift = (2.0 ** 0.5) * torch.distributions.Normal(0.0, 1.0).icdf(torch.tensor(c["p_attn"])).item()
    gen = torch.Generator().manual_seed(4000 + sid)
    x = torch.randn(1, L, H, V, generator=gen)
    dt = torch.nn.functional.softplus(torch.randn(1, L, H, generator=gen) - 2.0)
    k = (torch.randn(1, L, H, K, generator=gen) * K ** -0.5).bfloat16()
    q = (torch.randn(1, L, H, K, generator=gen) * K ** -0.5).bfloat16()
    logits = torch.randn(1, L // nbs, H, 2, generator=gen)
    logits[..., 0] += shift
    ty = torch.zeros_like(logits).scatter_(-1, logits.softmax(-1).max(-1, keepdim=True)[1], 1.0)
    if sid == n_glob - 1:
        ty[:, -1] = 1
    return dict(q=q, k=k, v=(x * dt[..., None]).bfloat16(), g=A.view(1, 1, H) * dt, types=ty)


def mamba_long_parity(o_m, o_a, ids, n_glob: int, L: int, heads: int = 2, win: int = 128):
    """Rank 0: regenerates the whole sequence on the host (every segment from its seed), evaluates the oracle for
    ``heads`` heads, and compares the last ``win`` tokens of this rank's last local segment (linear branch:
    chunk form over the whole sequence; softmax branch: masked SDPA for the window's queries against all keys)."""
    from oracle import attn as oattn
    from oracle import gdn as ogdn
    c = MAMBA_LONG
    T, K, nbs = c["T"], c["K"], c["nbs"]
    segs = [mamba_long_segment(sid, n_glob, L) for sid in range(n_glob)]
    cat = lambda n: torch.cat([sg[n][:, :, :heads] for sg in segs], 1)
    q, k, v = (cat(n).float().contiguous() for n in ("q", "k", "v"))
    g, types = cat("g").contiguous(), cat("types").contiguous()
    o_ref, _ = ogdn.linear_chunk(q, k, v, g, None, types[..., 1], nbs=nbs, scale=1.0, decay=True, use_l2norm=False,
                                 rule="mamba", reference_trailing_carry=False)
    t0 = (ids[-1] + 1) * L - win                                  # the last tokens of the rank's last segment (global)
    loc = len(ids) * L - win                                      # their position in this rank's tensors
    mask = oattn.attn_mask_rows(types[..., 0], T, nbs, heads, t0, t0 + win)
    oa_ref, _ = oattn.attn_sdpa(q[:, t0:t0 + win], k, v, mask, K ** -0.5)
    err_l = float((o_m[:, loc:loc + win, :heads].float().cpu() - o_ref[:, t0:t0 + win]).abs().max())
    err_a = float((o_a[:, loc:loc + win, :heads].float().cpu() - oa_ref).abs().max())
    mag = float(max(o_ref[:, t0:t0 + win].abs().max(), oa_ref.abs().max()))
    return {"max_abs_err_o_mamba": err_l, "max_abs_err_o_attn": err_a, "max_abs_ref": mag, "tolerance": "rtol=atol=1e-2",
            "sample": f"tokens {t0}..{t0 + win - 1}, heads 0..{heads - 1}, device outputs vs the fp32 CPU oracle over the whole sequence"}


def mamba_long_measure(args, rank: int, world: int, dev, group=None, lin_group=None, plan: bool = True,
                       parity: bool = True):
    """One measurement of the long-context NAtSL-Mamba2 layer (B=1, T=65536, H=32, state dim 128, head dim 64, block 256,
    ~10 % softmax blocks) split over the ``world`` ranks of ``group``; world = 1 runs the same op on one GPU (the
    recurrence cut into parallel sub-segments).  -> dict(ms_per_step, host_issue_ms_per_step, launch, parity (rank 0))."""
    import neuralattentionsearchlinear_b200 as nat
    from neuralattentionsearchlinear_b200 import sequence_parallel as sp
    c = MAMBA_LONG
    T, H, K, V, nbs = c["T"], c["H"], c["K"], c["V"], c["nbs"]
    layout = args.sp_layout if world > 1 else "contiguous"
    ids = sp.segment_ids(rank, world, layout)
    n_glob = world * len(ids)
    L = T // n_glob
    segs = [mamba_long_segment(sid, n_glob, L) for sid in ids]
    q, k, v, g, types = (torch.cat([sg[n] for sg in segs], 1).to(dev) for n in ("q", "k", "v", "g", "types"))
    stream = torch.cuda.current_stream(dev)
    kv_cap = None

    def step():
        if args.sp_plain_op and world == 1:               # the layer's plain op: serial recurrence over the whole sequence
            return nat.nats_mixed_attn_mamba(q, k, v, q, k, v, None, g, types, None, scale_attn=K ** -0.5, nats_block_size=nbs,
                                             ops_for_incomplete_chunks="all", output_final_state_mamba=True,
                                             decay_for_non_mamba_blocks=True)
        return sp.nats_mixed_attn_mamba_sp(q, k, v, q, k, v, g, types, nats_block_size=nbs, scale_attn=K ** -0.5,
                                           decay_for_non_mamba_blocks=True, layout=layout,
                                           linear_splits=args.sp_linear_splits or None, kv_capacity=kv_cap, group=group,
                                           linear_group=lin_group)

    def barrier():
        if world > 1:
            torch.distributed.barrier(group)
        torch.cuda.synchronize(dev)

    for _ in range(max(3, args.warmup)):
        out = step()
    barrier()
    run_step, mode = step, "eager, gather capacity read back every step (one host synchronisation)"
    if args.sp_fixed_capacity and world > 1:
        # gather capacity fixed to the exact maxima of this input (read back by the warm-up steps): no host read
        kv_cap = sp.last_kv_capacity
        mode = "eager, caller-given gather capacity (no host synchronisation)"
        for _ in range(3):
            out = step()
        barrier()
    if world == 1 and not args.sp_plain_op and not args.sp_eager_one_gpu:
        # one GPU: the whole step (no collective, no host read) replays from one CUDA graph, so that the figure is the
        # device time of the step and not the host's launch rate
        gr = torch.cuda.CUDAGraph()
        holder = {}
        with torch.cuda.graph(gr):
            holder["out"] = step()
        torch.cuda.synchronize(dev)

        def run_step():
            gr.replay()
            return holder["out"]
        mode = "one CUDA graph for the whole step"
        for _ in range(3):
            out = run_step()
        barrier()
    if plan and world > 1:
        # plan / replay: the compute stages replay from CUDA graphs, the all-gathers stay eager between them
        pl = sp.GraphedMambaSP(q, k, v, q, k, v, g, types, kv_capacity=sp.last_kv_capacity, nats_block_size=nbs,
                               scale_attn=K ** -0.5, decay_for_non_mamba_blocks=True, layout=layout,
                               linear_splits=args.sp_linear_splits or None, group=group, linear_group=lin_group,
                               gather_under_linear={"auto": None, "gather-under-linear": True,
                                                    "branches-side-by-side": False}[args.sp_plan_order])
        pl.capture()
        run_step = pl.run
        mode = ("plan: compute replayed from CUDA graphs, eager NCCL all-gathers between them, "
                + ("key/value gather under the linear branch" if pl.gather_under_linear else "branches side by side"))
        for _ in range(3):
            out = run_step()
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_host0 = time.perf_counter()
    e0.record(stream)
    for _ in range(args.steps):
        out = run_step()
    e1.record(stream)
    host_ms = (time.perf_counter() - t_host0) * 1e3 / args.steps      # host time to issue one step
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group)
        ms = float(t.item())
    res = {"ms_per_step": ms / args.steps, "tokens_per_s": T / (ms / args.steps * 1e-3), "host_issue_ms_per_step": host_ms,
           "launch": mode, "layout": layout}
    if parity and rank == 0:
        res["parity"] = mamba_long_parity(out[0], out[1], ids, n_glob, L)
    return res


def run_mamba_long(args, rank: int, world: int, local_rank: int):
    """``--workload mamba_long``: the long-context layer, sequence-parallel over the ranks (strong scaling)."""
    from neuralattentionsearchlinear_b200 import _lib
    _lib.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = init_process_group_quiet(dev) if world > 1 else None
    lin_group = dist.new_group() if dist is not None else None      # own communicator for the state exchange
    res = mamba_long_measure(args, rank, world, dev, group=None, lin_group=lin_group, plan=args.sp_plan)
    status = _lib.load().natsl_device_status()
    if rank == 0:
        print(json.dumps({"metric": "prefill_tokens_per_s", "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
                          "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": res["ms_per_step"],
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                          "data": "synthetic (seeded, generated per rank)",
                          "config": {"workload": "natsl_mamba2_layer_fwd B=1 T=65536 H=32 dstate=128 dhead=64 block=256 "
                                     "p_softmax=0.10", "parallelism": f"sequence-parallel x{world} ({res['layout']} segments)",
                                     "launch": res["launch"]},
                          "host_issue_ms_per_step": res["host_issue_ms_per_step"], "parity": res.get("parity"),
                          "device_status": status}))
    if dist is not None:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------- model-level workloads (optional)
MODEL_CFGS = {
    # 24 layers, hidden 1024, 16 heads of dim 64, SwiGLU 2816, vocab 32000, block 64; global batch 16 x 4096 (prefill)
    "model_prefill": dict(hidden_size=1024, head_dim=64, num_heads=16, num_attn_heads=16, global_batch=16, per_gpu_batch=None),
    # 1.3B: 24 layers, hidden 2048, 16 heads of dim 128, SwiGLU 5632; 8 x 4096 tokens per GPU, forward + backward
    "model_fwdbwd": dict(hidden_size=2048, head_dim=128, num_heads=16, num_attn_heads=16, global_batch=None, per_gpu_batch=8),
}


def run_model(args, rank: int, world: int, local_rank: int):
    """Decoder model around the NAtSL-GDN layer, random init (seed 0), uniform random token ids.
    model_prefill: bf16 forward under eval, global batch 16 split over the ranks (strong scaling, no collective).
    model_fwdbwd: forward + backward of the next-token loss under train, 8 sequences per GPU (weak scaling), gradients
    averaged with torch's bucketed NCCL all-reduce overlapped with the backward pass (DistributedDataParallel)."""
    from neuralattentionsearchlinear_b200 import _lib
    from neuralattentionsearchlinear_b200.models import (NeuralAttentionSearchLineraAttnGDNConfig,
                                                         NeuralAttentionSearchLinearAttnGDNForCausalLM)
    _lib.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = init_process_group_quiet(dev) if world > 1 else None
    mc = MODEL_CFGS[args.workload]
    train = args.workload == "model_fwdbwd"
    T = 4096
    layers = args.layers or 24
    cfg = NeuralAttentionSearchLineraAttnGDNConfig(
        hidden_size=mc["hidden_size"], expand_v=1.0, head_dim=mc["head_dim"], num_heads=mc["num_heads"],
        num_attn_heads=mc["num_attn_heads"], num_hidden_layers=layers, vocab_size=32000, nats_block_size=64,
        ops_for_incomplete_chunks="all", gdn_layers=[], attn_apply_pos_encoding=False, attn_qk_norm=True,
        attn_with_short_conv=True, decay_for_non_gdn_blocks=True, norm_eps=1e-6)
    torch.manual_seed(0)
    model = NeuralAttentionSearchLinearAttnGDNForCausalLM(cfg).to(dev).bfloat16()
    n_params = sum(p.numel() for p in model.parameters())
    if train:
        B = mc["per_gpu_batch"]
        model.train()
        net = model
        if dist is not None:
            net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], gradient_as_bucket_view=True)
    else:
        assert mc["global_batch"] % world == 0, "the global batch of 16 must divide over the ranks"
        B = mc["global_batch"] // world
        model.eval()
        net = model
    gen = torch.Generator().manual_seed(100 + rank)
    ids_host = torch.randint(0, 32000, (B, T), generator=gen).pin_memory()
    ids = ids_host.to(dev)
    stream = torch.cuda.current_stream(dev)

    def step(x):
        if train:
            net.zero_grad(set_to_none=True)
            out = net(input_ids=x, labels=x)
            out["loss"].backward()
            return out["loss"].detach()
        with torch.no_grad():
            return net(input_ids=x, logits_to_keep=1)["logits"]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    clocks = ClockSampler(vis.split(",")[local_rank].strip() if vis else local_rank)
    if rank == 0:
        clocks.start()
    for _ in range(max(3, args.warmup)):
        res = step(ids)
    barrier()
    if rank == 0:
        clocks.rows.clear()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        res = step(ids)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    # end to end: the token ids come from pinned host memory and the result (loss / last-token logits) goes back
    host_out = torch.empty_like(res, device="cpu").pin_memory()
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record(stream)
    for _ in range(args.steps):
        x = ids_host.to(dev, non_blocking=True)
        host_out.copy_(step(x), non_blocking=True)
    e3.record(stream)
    barrier()
    ms_e2e = e2.elapsed_time(e3)
    if dist is not None:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = (float(x) for x in t.tolist())
    clk = clocks.stop() if rank == 0 else None
    # share of the step spent in the hybrid attention op: the op alone on one layer's shapes, times the layer count
    import neuralattentionsearchlinear_b200 as nat
    H, D = mc["num_heads"], mc["head_dim"]
    g_ = torch.Generator(device=dev).manual_seed(1)
    rnd = lambda *sh: torch.randn(*sh, device=dev, generator=g_).bfloat16()
    q, k, v = rnd(B, T, H, D), rnd(B, T, H, D), rnd(B, T, H, D)
    gdec = -torch.nn.functional.softplus(torch.randn(B, T, H, device=dev, generator=g_))
    beta = torch.rand(B, T, H, device=dev, generator=g_).bfloat16()
    types = torch.zeros(B, T // 64, H, 2, device=dev)
    types[..., 1] = 1
    types[:, ::4, :, 0], types[:, ::4, :, 1] = 1, 0
    types[:, -1] = 1
    if train:
        q, k, v, gdec, beta = (x.requires_grad_(True) for x in (q, k, v, gdec, beta))

    def op_step():
        o_l, o_a, _ = nat.nats_mixed_attn_gdn(q, k, v, q, k, v, None, gdec, beta, types, None, nats_block_size=64,
                                              ops_for_incomplete_chunks="all", decay_for_non_gdn_blocks=True)
        if train:
            (o_l.float().sum() + o_a.float().sum()).backward()

    for _ in range(3):
        op_step()
    torch.cuda.synchronize(dev)
    e4, e5 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e4.record(stream)
    for _ in range(5):
        op_step()
    e5.record(stream)
    torch.cuda.synchronize(dev)
    op_ms = e4.elapsed_time(e5) / 5
    status = _lib.load().natsl_device_status()
    if rank == 0:
        ms_step = ms / args.steps
        tokens = world * B * T
        # dense FLOPs per token of the matrix products outside the hybrid op (projections, MLP, LM head for training)
        hs, inter = mc["hidden_size"], 256 * ((int(mc["hidden_size"] * 4 * 2 / 3) + 255) // 256)
        per_layer = 2 * hs * (3 * hs + hs + hs) + 2 * 3 * hs * inter
        dense = layers * per_layer + (2 * hs * 32000 if train else 0)
        mult = 3 if train else 1
        print(json.dumps({
            "metric": "train_tokens_per_s" if train else "prefill_tokens_per_s", "value": tokens / (ms_step * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak" if train else "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform random token ids, random-init weights, seed 0)",
            "config": {"workload": f"natsl_gdn_decoder {'fwd+bwd' if train else 'prefill'} layers={layers} hidden={hs} "
                                   f"heads={H}x{D} vocab=32000 block=64 T=4096", "per_gpu_batch": B, "parameters": n_params,
                       "parallelism": (f"data-parallel x{world}" + (", bucketed NCCL gradient all-reduce overlapped with backward"
                                                                   if train and world > 1 else ""))},
            "clocks": clk,
            "e2e": {"value": tokens / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * T * 8,
                    "d2h_bytes_per_step": host_out.numel() * host_out.element_size(), "ms_per_step": ms_e2e / args.steps},
            "hybrid_attention_op": {"ms_per_layer": op_ms, "share_of_step": layers * op_ms / ms_step,
                                    "note": "the op alone (forward" + (" + backward" if train else "") + ") on one layer's shapes x layers"},
            "dense_matmul_tflops_outside_op": mult * dense * tokens / world / (max(ms_step - layers * op_ms, 1e-6) * 1e-3) / 1e12,
            "device_status": status}))
    if dist is not None:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------- layer forward + backward (optional)
def run_layer_fwdbwd(args, rank: int, world: int, local_rank: int):
    """One step = forward + backward of ``nats_mixed_attn_gdn`` on the layer configuration (B=8, T=4096, H=16, d=128,
    block 64) with every differentiable input requiring a gradient; per-stage device times and rooflines of the backward
    kernels; gradients of a (sequence, head) sample checked against the oracle."""
    import neuralattentionsearchlinear_b200 as nat
    from neuralattentionsearchlinear_b200 import _lib, _ops
    _lib.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = init_process_group_quiet(dev) if world > 1 else None
    B, T, H, K, V, nbs = (CFG[n] for n in ("B", "T", "H", "K", "V", "nbs"))
    host = make_inputs(1000 * rank, B, H)
    gen = torch.Generator().manual_seed(77 + rank)
    do_l = torch.randn(B, T, H, V, generator=gen).bfloat16()
    do_a = torch.randn(B, T, H, V, generator=gen).bfloat16()
    leaf = lambda n: host[n].to(dev).requires_grad_(True)
    q, k, v, g, beta, types = (leaf(n) for n in ("q", "k", "v", "g", "beta", "types"))
    dl, da = do_l.to(dev), do_a.to(dev)
    stream = torch.cuda.current_stream(dev)

    def step():
        for t_ in (q, k, v, g, beta, types):
            t_.grad = None
        o_l, o_a, _ = nat.nats_mixed_attn_gdn(q, k, v, q, k, v, None, g, beta, types, None, nats_block_size=nbs,
                                              ops_for_incomplete_chunks="all", decay_for_non_gdn_blocks=True)
        torch.autograd.backward([o_l, o_a], [dl, da])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    clocks = ClockSampler(vis.split(",")[local_rank].strip() if vis else local_rank)
    if rank == 0:
        clocks.start()
    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize(dev)
    t_w = time.perf_counter()
    while time.perf_counter() - t_w < args.min_warm_seconds:
        for _ in range(5):
            step()
        torch.cuda.synchronize(dev)
    if rank == 0:
        clocks.rows.clear()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = _lib.kernel_launches()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    gpu_launches = _lib.kernel_launches() - launches_before
    barrier()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clk = clocks.stop() if rank == 0 else None
    ms_step = ms / args.steps
    # ---- per-stage device times of the backward pass (CUDA events around every C-ABI call)
    tb = nat.build_selection_tables(types.detach(), T, nbs)
    with torch.no_grad():
        o_attn, lse = _ops.attn_fwd(q, k, v, tb, K ** -0.5, True)
        timer = _ops.StageTimer()
        reps = max(3, min(args.steps, 10))
        for _ in range(reps):
            _ops.attn_bwd(q, k, v, o_attn, lse, da, tb, K ** -0.5, True, timer=timer)
            res = _ops.linear_bwd(_lib.RULE_GDN, q, k, v, g.detach(), beta.detach(), tb, K ** -0.5, None, True, True, dl, timer=timer)
        stage_ms = {n: t_ / reps for n, t_ in timer.result().items()}
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peaks = json.load(open(peaks_path))
        peak_tf, peak_bw, peak_src = float(peaks["bf16_tflops_sustained"]), float(peaks["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    else:
        peak_tf, peak_bw, peak_src = 1400.0, 6650.0, "fallback"
    n_tok = B * T * H
    NT = T // 64
    st_b = B * NT * H * K * V * 2                         # one K x V bf16 state per chunk
    frac_lin = float(host["types"][..., 1].float().mean())
    work = {
        # five products per visible (query chunk, key chunk) pair: S, dP, dQ, dK, dV
        "attn_bwd": ("tensor", 2.5 * attention_tile_flops(host["types"], H, K, V), "attn_bwd_dq_kernel + attn_bwd_dkdv_kernel"),
        "recompute_prep": ("hbm", n_tok * (K + V) * 2 + n_tok * (K + V) * 2 + n_tok * 14, "gdn_prep_kernel<128,128>"),
        "recompute_scan": ("hbm", frac_lin * n_tok * (2 * K + V) * 2 + st_b, "linear_scan_kernel<128,32,gdn>"),
        "bwd_pre": ("hbm", n_tok * (2 * K + V) * 2 + n_tok * (2 * K + V) * 2, "linear_bwd_pre_kernel<128,128>"),
        "bwd_dh": ("hbm", n_tok * (3 * K + 2 * V) * 2 + frac_lin * st_b + n_tok * V * 2, "linear_bwd_dh_kernel<128,32,gdn>"),
        "bwd_state": ("hbm", n_tok * (2 * K + 3 * V) * 2 + st_b + frac_lin * st_b + n_tok * (3 * K + V) * 2,
                      "linear_bwd_state_kernel<128,128,gdn>"),
        "bwd_intra": ("hbm", n_tok * (6 * K + 5 * V) * 2 + n_tok * (2 * K + V) * 2, "linear_bwd_intra_kernel<128,128,gdn>"),
        "bwd_dg": ("hbm", n_tok * 8 + B * NT * H * 16, "linear_bwd_dg_kernel"),
    }
    roofs = {}
    for n, (bound, amount, kname) in work.items():
        sec = stage_ms[n] * 1e-3
        ach, peak, unit = (amount / sec / 1e12, peak_tf, "TFLOP/s") if bound == "tensor" else (amount / sec / 1e9, peak_bw, "GB/s")
        roofs[n] = {"kernel": kname, "bound": bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                    "traffic": None, "algorithmic_per_launch": amount, "ms_per_launch": stage_ms[n]}
    dom = max(stage_ms, key=lambda n: stage_ms[n])
    # ---- parity of the timed gradients: one sequence, a few heads, against the oracle in float64
    from oracle import grad as ograd
    hs = 2
    sl = lambda x: x[:1, :, :hs].detach().double().cpu().contiguous()
    ty = host["types"][:1, :, :hs].float()
    ra = ograd.attn_grads(sl(q), sl(k), sl(v), ty[..., 0], do_a[:1, :, :hs].double(), nbs=nbs)
    rl = ograd.linear_chunk_backward(sl(q), sl(k), sl(v), sl(g), sl(beta), ty[..., 1], do_l[:1, :, :hs].double(), None, decay=True)
    got_q = q.grad[:1, :, :hs].double().cpu()
    ref_q = ra["dq"] + rl["dq"]
    got_g, ref_g = g.grad[:1, :, :hs].double().cpu(), rl["dg"]
    par = {"max_abs_err_dq": float((got_q - ref_q).abs().max()), "max_abs_dq": float(ref_q.abs().max()),
           "max_abs_err_dg": float((got_g - ref_g).abs().max()), "max_abs_dg": float(ref_g.abs().max()),
           "sample": f"sequence 0, heads 0..{hs - 1}: dq (both branches) and dg of the timed step vs the float64 CPU oracle"}
    print(json.dumps({
        "metric": "train_tokens_per_s", "value": world * B * T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded, generated on the host)",
        "config": {"workload": "natsl_gdn_layer_fwd+bwd B={} T=4096 H=HQ=16 dk=dv=128 block=64 bf16 p_softmax=0.25".format(B),
                   "per_gpu_batch": B, "parallelism": f"replicas x{world} (batch sharded, no collective)"},
        "clocks": clk, "gpu_launches": gpu_launches, "kernel_ms": stage_ms,
        "roofline": dict(roofs[dom], peak_source=peak_src, dominant_stage=dom), "roofline_all": roofs, "parity": par}))
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=CFG["B"], help="sequences per GPU (default: the benchmark's 8; "
                    "smaller values are for profiler captures only)")
    ap.add_argument("--min-warm-seconds", type=float, default=1.5, help="minimum warm-up time under load")
    ap.add_argument("--sp-layout", default="zigzag", choices=["contiguous", "zigzag"],
                    help="segment layout of the sequence-parallel workload (mamba_long)")
    ap.add_argument("--sp-linear-splits", type=int, default=0,
                    help="sub-segments per segment in the linear branch of mamba_long (0: about 1024 tokens each)")
    ap.add_argument("--sp-plan", action="store_true",
                    help="mamba_long on several GPUs through the plan / replay form (CUDA graphs for the compute stages)")
    ap.add_argument("--sp-plan-order", default="auto", choices=["auto", "gather-under-linear", "branches-side-by-side"])
    ap.add_argument("--sp-fixed-capacity", action="store_true",
                    help="mamba_long: size the key/value gather from a capacity fixed before the timed region instead of "
                         "reading the block counts back every step")
    ap.add_argument("--sp-eager-one-gpu", action="store_true",
                    help="mamba_long on one GPU: issue the step eagerly instead of replaying it from a CUDA graph")
    ap.add_argument("--sp-plain-op", action="store_true",
                    help="mamba_long on one GPU through nats_mixed_attn_mamba (no sub-segment split, one stream)")
    ap.add_argument("--workload", default="gdn_layer", choices=["gdn_layer", "gdn_layer_fwdbwd", "mamba_long", "model_prefill", "model_fwdbwd"],
                    help="gdn_layer: the headline single-GPU layer configuration (default); mamba_long: the long-context "
                         "Mamba2 layer, sequence-parallel over the ranks; model_prefill / model_fwdbwd: the 24-layer "
                         "decoder models (prefill of 16 x 4096 tokens; forward + backward of 8 x 4096 tokens per GPU)")
    ap.add_argument("--no-graph", action="store_true",
                    help="default workload: time the eagerly issued step instead of its CUDA-graph replay")
    ap.add_argument("--no-sp", action="store_true",
                    help="gdn_layer with N > 1: leave out the sequence-parallel long-context measurement (sp_long_context)")
    ap.add_argument("--layers", type=int, default=0, help="model workloads: number of layers (default 24)")
    args = ap.parse_args()
    CFG["B"] = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.impl == "reference":
        run_reference(args, rank)
    elif args.workload == "mamba_long":
        run_mamba_long(args, rank, world, local_rank)
    elif args.workload == "gdn_layer_fwdbwd":
        run_layer_fwdbwd(args, rank, world, local_rank)
    elif args.workload in MODEL_CFGS:
        run_model(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
