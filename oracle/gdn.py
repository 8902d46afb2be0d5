"""Oracle (test infrastructure): the linear-attention branch (Gated DeltaNet, and
Mamba2/SSD through ``rule='mamba'``) with per-(block, head) selection.

Two independent CPU forms are given and cross-checked by the tests:

``linear_recurrent``  token-by-token recurrence with re-roll to the block-start
    state when the finished block was not selected.  Restates
    src/nats/ops/gated_delta_rule/fused_recurrent.py:160-300 (per-token update
    order: decay, delta-rule write, read) together with the re-roll loop of the
    reference's own debug script, fused_recurrent.py:754-785; Mamba2 twin:
    src/nats/ops/mamba/fused_recurrent.py:121-322.

``linear_chunk``  64-token chunk form following the reference's chunk kernels:
    chunk-local cumsum of the log decay plus the carry of skipped blocks
    (src/nats/ops/utils/cumsum.py:85-133), A = strictLower(beta k k^T Gamma)
    (src/nats/ops/common/chunk_scaled_dot_kkt.py:105-126), (I+A)^-1
    (src/nats/ops/utils/solve_tril.py:350-447), w/u
    (src/nats/ops/gated_delta_rule/wy_fast.py:123-153), the state recurrence over
    selected chunks (src/nats/ops/common/chunk_delta_h.py:189-324) and the output
    of every chunk (src/nats/ops/common/chunk_o.py:124-215); Mamba2:
    src/nats/ops/mamba/chunk_h.py:139-218, src/nats/ops/mamba/chunk_o.py:137-198.

Conventions: q, k [B,T,H,K]; v [B,T,H,V]; g, beta [B,T,H]; ``sel`` [B,TN,HN] is
column 1 of the block types (1 = this block updates the recurrent state); linear
head h uses selection head ``h // (H // HN)`` (chunk_delta_h.py:83-84).  Mode
``ops_for_incomplete_chunks='all'`` with ``incomplete_block_start_with_ht=True``.

The carry of skipped blocks is kept as a separate scalar per chunk; because the
inverse and the intra-chunk score matrix only use decay *differences*, the
reference's ``w`` (computed from the carried cumsum) equals ``exp(carry) * w_local``.

Reference quirk kept on purpose (``reference_trailing_carry=True``): the carry
kernel is launched per *selected* chunk and fills the skipped chunks before it
(cumsum.py:95-133), so skipped blocks after the last selected block get no carry.
The layer always forces the last block to be selected
(src/nats/layers/natsl_attn_gdn.py:553), where this makes no difference.

For ``nats_block_size > 64`` the reference's chunk kernels are not
self-consistent (its own notes: src/nats/ops/gated_delta_rule/chunk.py:47-50);
the chunk form here follows the token recurrence instead: the 64-token sub-chunks
of an unselected block update a temporary state that is rolled back at the end
of the block.

``own_chunk=False`` is the mode in which only the softmax branch covers the current
chunk (``ops_for_incomplete_chunks='attn'``, src/nats/ops/mixed_ops/mixed_attn_gdn.py:35-42,86):
the output keeps just the state term, o = scale * e^{g} q S with S the state after the
most recent selected 64-token chunk (src/nats/ops/common/chunk_o.py:210-211), and the
selection acts per 64-token chunk (every chunk of a selected block updates the state,
chunks of an unselected block only decay it), which is how the reference's chunk
kernels walk in this mode (chunk_delta_h.py:189-324 iterates selected chunks).
"""
from __future__ import annotations

import torch

CHUNK = 64


def l2norm(x: torch.Tensor) -> torch.Tensor:
    """x * rsqrt(sum x^2 + 1e-6) over the last axis (fused_recurrent.py:166-169)."""
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def _expand_sel(sel: torch.Tensor, H: int) -> torch.Tensor:
    B, TN, HN = sel.shape
    assert H % HN == 0
    return sel.to(torch.bool).repeat_interleave(H // HN, dim=2)          # [B,TN,H]


def _per_chunk_selection(sel, nbs, T):
    """[B,TN,HN] per block -> [B,NT,HN] per 64-token chunk."""
    NT = -(-T // CHUNK)
    return sel.repeat_interleave(nbs // CHUNK, dim=1)[:, :NT]


def linear_recurrent(q, k, v, g, beta, sel, nbs=64, scale=None, h0=None, decay=True,
                     use_l2norm=True, rule="gdn", own_chunk=True, return_block_start=False):
    """Token recurrence with re-roll.  Returns (o [B,T,H,V], final_state [B,H,K,V]).

    final_state is the state at the end of the last selected block (what the
    reference's chunk recurrence holds when it stops, chunk_delta_h.py:311-324).
    With ``return_block_start`` a third value is returned: the state a decoder
    continues from (src/nats/ops/gated_delta_rule/chunk_fwd.py:178-206) -- when T ends
    a block, the state after that block's end-of-block step (kept if the block
    is selected in ``sel``, else rolled back); otherwise the state at the start
    of the unfinished last block.
    """
    B, T, H, K = q.shape
    V = v.shape[-1]
    dt = q.dtype
    if scale is None:
        scale = K ** -0.5
    if use_l2norm:
        q, k = l2norm(q), l2norm(k)
    if not own_chunk:
        sel, nbs = _per_chunk_selection(sel, nbs, T), CHUNK
    selh = _expand_sel(sel, H)
    S = torch.zeros(B, H, K, V, dtype=dt) if h0 is None else h0.to(dt).clone()
    S0 = S.clone()
    Sfin = S.clone()
    gsum = torch.zeros(B, H, dtype=dt)
    o = torch.zeros(B, T, H, V, dtype=dt)
    for t in range(T):
        gt = g[:, t].to(dt)
        S = S * gt.exp()[..., None, None]
        gsum = gsum + gt
        kt = k[:, t]
        if rule == "gdn":
            vt = beta[:, t].to(dt)[..., None] * (v[:, t] - torch.einsum("bhkv,bhk->bhv", S, kt))
        else:
            vt = v[:, t]
        S = S + kt[..., :, None] * vt[..., None, :]
        S_read = S if own_chunk else S0 * gsum.exp()[..., None, None]      # chunk-start state, decayed to t
        o[:, t] = torch.einsum("bhkv,bhk->bhv", S_read, q[:, t] * scale)
        if (t + 1) % nbs == 0 or t == T - 1:
            if t == T - 1 and (t + 1) % nbs != 0:
                start = S0.clone()                       # start of the unfinished block
            m = selh[:, t // nbs][..., None, None]
            rolled = S0 * gsum.exp()[..., None, None] if decay else S0
            S = torch.where(m, S, rolled)
            Sfin = torch.where(m, S, Sfin)
            S0 = S.clone()
            gsum = torch.zeros_like(gsum)
            if t == T - 1 and (t + 1) % nbs == 0:
                start = S0.clone()
    if return_block_start:
        return o, Sfin, start
    return o, Sfin


def linear_chunk(q, k, v, g, beta, sel, nbs=64, scale=None, h0=None, decay=True,
                 use_l2norm=True, rule="gdn", reference_trailing_carry=True,
                 return_intermediates=False, own_chunk=True):
    """Chunk form (64-token compute chunks).  Same returns as ``linear_recurrent``;
    with ``return_intermediates`` also a dict of per-chunk tensors:
    gcs [B,T,H] (chunk-local cumsum), k_rstd [B,T,H], w [B,T,H,K], u [B,T,H,V]
    (carry-free) and h [B,NT,H,K,V] (the state each chunk reads) and
    carry [B,NT,H].
    """
    B, T, H, K = q.shape
    V = v.shape[-1]
    dt = q.dtype
    C = CHUNK
    assert nbs % C == 0
    if not own_chunk:
        sel, nbs = _per_chunk_selection(sel, nbs, T), C
    cpb = nbs // C
    if scale is None:
        scale = K ** -0.5
    k_rstd = torch.rsqrt((k * k).sum(-1) + 1e-6) if use_l2norm else torch.ones(B, T, H, dtype=dt)
    if use_l2norm:
        q, k = l2norm(q), l2norm(k)
    NT = -(-T // C)
    Tp = NT * C

    def pad(x):
        if Tp == T:
            return x
        z = torch.zeros((B, Tp - T) + tuple(x.shape[2:]), dtype=x.dtype)
        return torch.cat([x, z], 1)

    if beta is None:
        beta = torch.ones(B, T, H, dtype=dt)
    qp, kp, vp, gp, bp = (pad(x.to(dt)) for x in (q, k, v, g, beta))
    # [B,H,NT,C,*]
    qc = qp.view(B, NT, C, H, K).permute(0, 3, 1, 2, 4)
    kc = kp.view(B, NT, C, H, K).permute(0, 3, 1, 2, 4)
    vc = vp.view(B, NT, C, H, V).permute(0, 3, 1, 2, 4)
    gc = gp.view(B, NT, C, H).permute(0, 3, 1, 2).cumsum(-1)            # chunk-local cumsum
    bc = bp.view(B, NT, C, H).permute(0, 3, 1, 2)
    gam = (gc[..., :, None] - gc[..., None, :])
    tril_s = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)
    tril_i = torch.tril(torch.ones(C, C, dtype=torch.bool), 0)
    kk = kc @ kc.transpose(-1, -2)
    if rule == "gdn":
        A = torch.where(tril_s, bc[..., :, None] * kk * gam.exp(), torch.zeros((), dtype=dt))
        eye = torch.eye(C, dtype=dt)
        Ai = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
        u = Ai @ (vc * bc[..., None])
        w = Ai @ (kc * (bc * gc.exp())[..., None])
    else:
        u = vc
        w = torch.zeros_like(kc)
    P = torch.where(tril_i, (qc @ kc.transpose(-1, -2)) * gam.exp(), torch.zeros((), dtype=dt))
    gL = gc[..., -1]                                                    # [B,H,NT]

    selh = _expand_sel(sel, H).permute(0, 2, 1)                         # [B,H,TN]
    TN = selh.shape[-1]
    idx = torch.arange(TN).view(1, 1, TN)
    last_sel = torch.where(selh, idx, torch.full_like(idx, -1)).amax(-1)  # [B,H], -1 if none

    S = torch.zeros(B, H, K, V, dtype=dt) if h0 is None else h0.to(dt).clone()
    Sfin = S.clone()
    carry = torch.zeros(B, H, dtype=dt)
    S_save, carry_save, blk_g = S.clone(), carry.clone(), torch.zeros(B, H, dtype=dt)
    o = torch.zeros(B, H, NT, C, V, dtype=dt)
    h_all = torch.zeros(B, NT, H, K, V, dtype=dt)
    carry_all = torch.zeros(B, NT, H, dtype=dt)
    for c in range(NT):
        blk, sub = c // cpb, c % cpb
        s_c = selh[..., blk]                                            # [B,H]
        may_carry = (blk < last_sel) if reference_trailing_carry else torch.ones_like(s_c)
        may_carry = may_carry & bool(decay)
        if sub == 0:
            S_save, carry_save, blk_g = S.clone(), carry.clone(), torch.zeros_like(carry)
        h_all[:, c] = S
        carry_all[:, c] = carry
        ec = carry.exp()[..., None, None]
        vprime = u[:, :, c] - ec * (w[:, :, c] @ S)                      # chunk_delta_h.py:218-234 / chunk_o.py:167-171,206-208
        o[:, :, c] = scale * (gc[:, :, c] + carry[..., None]).exp()[..., None] * (qc[:, :, c] @ S)
        if own_chunk:
            o[:, :, c] = o[:, :, c] + scale * (P[:, :, c] @ vprime)        # chunk_o.py:173,186,209 (else :210-211)
        gl = gL[:, :, c]
        if rule == "gdn":
            kdec = (gl[..., None] - gc[:, :, c]).exp()                   # chunk_delta_h.py:252
        else:
            kdec = torch.clamp(gl[..., None] - gc[:, :, c], max=0.0).exp()  # mamba/chunk_h.py:177
        S_new = (gl + carry).exp()[..., None, None] * S + kc[:, :, c].transpose(-1, -2) @ (vprime * kdec[..., None])
        blk_g = blk_g + gl
        if cpb == 1:
            act = s_c
            S = torch.where(act[..., None, None], S_new, S)
            carry = torch.where(act, torch.zeros_like(carry), torch.where(may_carry, carry + gl, carry))
            Sfin = torch.where(act[..., None, None], S, Sfin)
        else:
            S, carry = S_new, torch.zeros_like(carry)
            if sub == cpb - 1 or c == NT - 1:
                keep = s_c[..., None, None]
                S = torch.where(keep, S, S_save)
                carry = torch.where(s_c, carry, torch.where(may_carry, carry_save + blk_g, carry_save))
                Sfin = torch.where(keep, S, Sfin)
    o = o.permute(0, 2, 3, 1, 4).reshape(B, Tp, H, V)[:, :T]
    if not return_intermediates:
        return o, Sfin

    def unchunk(x, D=None):
        if D is None:
            return x.permute(0, 2, 3, 1).reshape(B, Tp, H)[:, :T]
        return x.permute(0, 2, 3, 1, 4).reshape(B, Tp, H, D)[:, :T]

    inter = dict(gcs=unchunk(gc), k_rstd=k_rstd, w=unchunk(w, K), u=unchunk(u, V), h=h_all,
                 carry=carry_all)
    return o, Sfin, inter
