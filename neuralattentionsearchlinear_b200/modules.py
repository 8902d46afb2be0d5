"""Small host-side modules the NAtSL layers are built from, restated in plain PyTorch (the reference
takes them from flash-linear-attention's Triton modules): RMSNorm, L2Norm, ShortConvolution,
mean pooling, the hard selection, and the two-input gated norm whose forward runs the CUDA kernel
``natsl_norm_gate_mix``.  Parameter names match the reference so state dicts load unchanged.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from .nats_util import current_stream_ptr


_ROW_WIDTHS = (64, 128, 256, 512, 1024, 2048)


def _dt(t):
    return _lib.DT_BF16 if (t is not None and t.dtype == torch.bfloat16) else _lib.DT_F32


def _kernel_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def _n_part(rows: int) -> int:
    return int(min(-(-rows // 8), 1184))


class _RMSNormFn(torch.autograd.Function):
    """``natsl_rmsnorm_fwd`` / ``natsl_rmsnorm_bwd`` on [rows, D] bf16: (y, s) with s = x (+ residual)."""

    @staticmethod
    def forward(ctx, x, residual, weight, eps):
        rows, D = x.shape
        y = torch.empty_like(x)
        s = torch.empty_like(x) if residual is not None else x
        _lib.call("natsl_rmsnorm_fwd", x.data_ptr(), _lib.ptr(residual), _lib.ptr(weight), _dt(weight), y.data_ptr(),
                  s.data_ptr() if residual is not None else None, rows, D, float(eps), current_stream_ptr(x.device))
        ctx.save_for_backward(s, weight)
        ctx.eps, ctx.has_res = float(eps), residual is not None
        return y, (s if residual is not None else None)

    @staticmethod
    def backward(ctx, dy, ds):
        s, weight = ctx.saved_tensors
        rows, D = s.shape
        dy = dy.contiguous()
        dadd = ds.contiguous() if (ctx.has_res and ds is not None) else None
        dx = torch.empty_like(s)
        n_part = _n_part(rows)
        dw_part = torch.empty(n_part, D, dtype=torch.float32, device=s.device)
        _lib.call("natsl_rmsnorm_bwd", s.data_ptr(), _lib.ptr(weight), _dt(weight), dy.data_ptr(), _lib.ptr(dadd), dx.data_ptr(),
                  dw_part.data_ptr(), n_part, rows, D, ctx.eps, current_stream_ptr(s.device))
        dw = None if weight is None else dw_part.sum(0).to(weight.dtype)
        return dx, (dx if ctx.has_res else None), dw, None


class RMSNorm(nn.Module):
    """y = x * rsqrt(mean(x^2) + eps) * weight (call sites: src/nats/layers/natsl_attn_gdn.py:233-235).  With
    ``(x, residual, True)`` it returns ``(norm(x + residual), x + residual)``, the fused pre-norm residual of
    src/nats/models/natsl_attn_gdn/modeling_natsl_attn_gdn.py:138-139.  CUDA bf16 inputs run ``natsl_rmsnorm_fwd`` /
    ``natsl_rmsnorm_bwd``; other inputs take the same expression in PyTorch."""

    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x, residual=None, prenorm: bool = False):
        D = x.shape[-1]
        if _kernel_ok(x) and D in _ROW_WIDTHS and self.weight.dtype in (torch.bfloat16, torch.float32):
            xr = x.contiguous().view(-1, D)
            rr = None if residual is None else residual.to(x.dtype).contiguous().view(-1, D)
            y, s = _RMSNormFn.apply(xr, rr, self.weight, self.eps)
            y = y.view(x.shape)
            return (y, s.view(x.shape)) if prenorm else y
        if residual is not None:
            x = (x + residual).to(x.dtype)
        xf = x.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)
        return (y, x) if prenorm else y


class L2Norm(nn.Module):
    """y = x * rsqrt(sum(x^2) + eps) (src/nats/layers/natsl_attn_mamba2.py:193-194)."""

    def __init__(self, eps: float = 1e-6):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + self.eps)).to(x.dtype)


class _ShortConvFn(torch.autograd.Function):
    """``natsl_short_conv_fwd`` / ``natsl_short_conv_bwd``: x [B,T,D] bf16, weight [D,1,W], bias [D] or None."""
    SPAN = 64            # tokens per partial weight sum; 64 selects the shared-memory tile kernel

    @staticmethod
    def forward(ctx, x, weight, bias, silu):
        B, T, D = x.shape
        W = weight.shape[-1]
        y = torch.empty_like(x)
        w2 = weight.reshape(D, W).to(torch.bfloat16).contiguous()
        b2 = None if bias is None else bias.to(torch.bfloat16).contiguous()
        _lib.call("natsl_short_conv_fwd", x.data_ptr(), w2.data_ptr(), _lib.ptr(b2), y.data_ptr(), B, T, D, W, int(silu),
                  current_stream_ptr(x.device))
        ctx.save_for_backward(x, weight, bias)
        ctx.silu = int(silu)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias = ctx.saved_tensors
        B, T, D = x.shape
        W = weight.shape[-1]
        dy = dy.contiguous()
        w2 = weight.reshape(D, W).to(torch.bfloat16).contiguous()
        b2 = None if bias is None else bias.to(torch.bfloat16).contiguous()
        span = _ShortConvFn.SPAN
        dx = torch.empty_like(x)
        dw_part = torch.empty(B * (-(-T // span)), D, W + 1, dtype=torch.float32, device=x.device)
        _lib.call("natsl_short_conv_bwd", x.data_ptr(), w2.data_ptr(), _lib.ptr(b2), dy.data_ptr(), dx.data_ptr(),
                  dw_part.data_ptr(), B, T, D, W, ctx.silu, span, current_stream_ptr(x.device))
        dw = dw_part.sum(0)
        dweight = dw[:, :W].reshape(weight.shape).to(weight.dtype)
        dbias = None if bias is None else dw[:, W].to(bias.dtype)
        return dx, dweight, dbias, None


class ShortConvolution(nn.Conv1d):
    """Depthwise causal conv1d over time followed by SiLU; returns (y, final_state)
    (src/nats/layers/natsl_attn_gdn.py:329-348, 430-447).  x: [B, T, D].  CUDA bf16 inputs with kernel size 4 run
    ``natsl_short_conv_fwd`` / ``natsl_short_conv_bwd`` (with a cache: over the cached tail followed by the new tokens);
    other inputs take PyTorch's conv1d."""

    def __init__(self, hidden_size: int, kernel_size: int, bias: bool = False, activation: Optional[str] = 'silu'):
        super().__init__(hidden_size, hidden_size, kernel_size, groups=hidden_size, bias=bias, padding=kernel_size - 1)
        self.hidden_size = hidden_size
        self.activation = activation

    def forward(self, x, cache=None, output_final_state=False, cu_seqlens=None):
        if cu_seqlens is not None:
            raise NotImplementedError("variable-length batches are not built")
        B, T, D = x.shape
        W = self.kernel_size[0]
        silu = self.activation in ('silu', 'swish')
        final = None
        if output_final_state:
            xt = x.transpose(1, 2)
            if cache is not None:
                xt = torch.cat([cache.to(xt.dtype), xt], -1)
            final = F.pad(xt, (max(0, W - xt.shape[-1]), 0))[..., -W:].contiguous()
        if _kernel_ok(x) and W == 4 and D % 8 == 0:
            if cache is None:
                return _ShortConvFn.apply(x.contiguous(), self.weight, self.bias, silu), final
            # decoding: the cached tail in front of the new tokens, so that every output is computed from the same four
            # inputs in the same order as in a one-shot pass (bit-identical q, k, v between the two)
            xc = torch.cat([cache[..., 1 - W:].transpose(1, 2).to(x.dtype), x], 1).contiguous()
            return _ShortConvFn.apply(xc, self.weight, self.bias, silu)[:, W - 1:].contiguous(), final
        xt = x.transpose(1, 2)
        if cache is not None:
            xt = torch.cat([cache.to(xt.dtype), xt], -1)
            y = F.conv1d(xt, self.weight, self.bias, groups=D)[..., -T:]
        else:
            y = F.conv1d(xt, self.weight, self.bias, padding=W - 1, groups=D)[..., :T]
        if silu:
            y = F.silu(y)
        return y.transpose(1, 2).contiguous(), final


class _BlockMeanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, nbs):
        B, T, D = x.shape
        NB = -(-T // nbs)
        y = torch.empty(B, NB, D, dtype=x.dtype, device=x.device)
        _lib.call("natsl_block_mean", x.data_ptr(), y.data_ptr(), B, T, D, int(nbs), current_stream_ptr(x.device))
        ctx.T, ctx.nbs = T, int(nbs)
        return y

    @staticmethod
    def backward(ctx, dy):
        T, nbs = ctx.T, ctx.nbs
        NB = dy.shape[1]
        cnt = torch.full((NB,), float(nbs), device=dy.device)
        cnt[-1] = T - (NB - 1) * nbs
        dx = (dy.float() / cnt.view(1, NB, 1)).to(dy.dtype).repeat_interleave(nbs, dim=1)[:, :T]
        return dx.contiguous(), None


def mean_pooling(x: torch.Tensor, chunk_size: int, cu_seqlens=None) -> torch.Tensor:
    """Per-chunk mean over time of x [B, T, H, D] -> [B, cdiv(T, chunk), H, D], fp32 sum divided by the number
    of tokens in the chunk (src/nats/ops/utils/pooling.py:51-57, call natsl_attn_gdn.py:412-416)."""
    if cu_seqlens is not None:
        raise NotImplementedError("variable-length batches are not built")
    B, T, H, D = x.shape
    NT = -(-T // chunk_size)
    if _kernel_ok(x) and (H * D) % 8 == 0:
        return _BlockMeanFn.apply(x.contiguous().view(B, T, H * D), chunk_size).view(B, NT, H, D)
    pad = NT * chunk_size - T
    xf = F.pad(x.float(), (0, 0, 0, 0, 0, pad)).view(B, NT, chunk_size, H, D).sum(2)
    cnt = torch.full((NT,), float(chunk_size), device=x.device)
    if pad:
        cnt[-1] = chunk_size - pad
    return (xf / cnt.view(1, NT, 1, 1)).to(x.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        y = torch.empty_like(a)
        _lib.call("natsl_swiglu_fwd", a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), current_stream_ptr(a.device))
        ctx.save_for_backward(a, b)
        return y

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        dy = dy.contiguous()
        da, db = torch.empty_like(a), torch.empty_like(b)
        _lib.call("natsl_swiglu_bwd", a.data_ptr(), b.data_ptr(), dy.data_ptr(), da.data_ptr(), db.data_ptr(), a.numel(),
                  current_stream_ptr(a.device))
        return da, db


def swiglu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """silu(a) * b (the activation of the reference's GatedMLP)."""
    if _kernel_ok(a) and b.dtype == a.dtype and a.numel() % 8 == 0 and a.shape == b.shape:
        return _SwiGLUFn.apply(a.contiguous(), b.contiguous())
    return F.silu(a) * b


def hard_softmax(logits: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """One-hot of the first maximum of softmax(logits) with a straight-through gradient
    (src/nats/layers/natsl_attn_gdn.py:47-61)."""
    y_soft = logits.softmax(dim)
    index = y_soft.max(dim, keepdim=True)[1]
    y_hard = torch.zeros_like(logits, memory_format=torch.legacy_contiguous_format).scatter_(dim, index, 1.0)
    return y_hard - y_soft.detach() + y_soft


class _NormGateMix(torch.autograd.Function):
    """y = (rms(x1) w1 a + rms(x2) w2 b) * act(g) on [rows, D] bf16 tensors: ``natsl_norm_gate_mix`` forward,
    ``natsl_norm_gate_mix_bwd`` backward (src/nats/modules/fused_norm_gate.py:38-182, 353, 657)."""

    @staticmethod
    def forward(ctx, x1, x2, g, xw, w1, w2, eps, activation):
        rows, D = x1.shape
        y = torch.empty_like(x1)
        _lib.call("natsl_norm_gate_mix", x1.data_ptr(), x2.data_ptr(), g.data_ptr(), _lib.ptr(xw), _dt(xw),
                  _lib.ptr(w1), _lib.ptr(w2), _dt(w1), y.data_ptr(), rows, D, float(eps), int(activation),
                  current_stream_ptr(x1.device))
        ctx.save_for_backward(x1, x2, g, xw, w1, w2)
        ctx.eps, ctx.activation = float(eps), int(activation)
        return y

    @staticmethod
    def backward(ctx, dy):
        x1, x2, g, xw, w1, w2 = ctx.saved_tensors
        rows, D = x1.shape
        dy = dy.contiguous()
        dx1, dx2, dg = torch.empty_like(x1), torch.empty_like(x2), torch.empty_like(g)
        dxw = torch.empty(rows, 2, dtype=torch.float32, device=x1.device) if xw is not None else None
        n_part = int(min(-(-rows // 8), 1184))
        dw_part = torch.empty(n_part, 2, D, dtype=torch.float32, device=x1.device)
        _lib.call("natsl_norm_gate_mix_bwd", x1.data_ptr(), x2.data_ptr(), g.data_ptr(), _lib.ptr(xw), _dt(xw),
                  _lib.ptr(w1), _lib.ptr(w2), _dt(w1), dy.data_ptr(), dx1.data_ptr(), dx2.data_ptr(), dg.data_ptr(),
                  _lib.ptr(dxw), dw_part.data_ptr(), n_part, rows, D, ctx.eps, ctx.activation, current_stream_ptr(x1.device))
        dw1 = dw2 = None
        if w1 is not None:
            dw = dw_part.sum(0)
            dw1, dw2 = dw[0].to(w1.dtype), dw[1].to(w2.dtype)
        return dx1, dx2, dg, (None if xw is None else dxw.to(xw.dtype)), dw1, dw2, None, None


class FusedMultiInputRMSNormGated(nn.Module):
    """y = (rms(x1) w1 a + rms(x2) w2 b) * g * sigmoid(g)  (src/nats/modules/fused_norm_gate.py:1354-1429).
    Runs ``natsl_norm_gate_mix`` (and its backward kernel) on CUDA bf16 inputs."""

    def __init__(self, hidden_size: int, elementwise_affine: bool = True, eps: float = 1e-5, activation: str = 'swish',
                 device=None, dtype=None):
        super().__init__()
        if activation not in ('swish', 'silu', 'sigmoid'):
            raise ValueError(f"Unsupported activation: {activation}")
        self.hidden_size, self.eps, self.activation = hidden_size, eps, activation
        if elementwise_affine:
            self.weight1 = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
            self.weight2 = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        else:
            self.register_parameter("weight1", None)
            self.register_parameter("weight2", None)

    def forward(self, x1, x2, g, x_weights_after_norm=None, residual=None, prenorm=False, residual_in_fp32=False):
        if residual is not None or prenorm:
            raise NotImplementedError("residual / prenorm variants are not built")
        D = self.hidden_size
        if not (x1.is_cuda and x1.dtype == torch.bfloat16):
            raise TypeError("FusedMultiInputRMSNormGated needs CUDA bf16 inputs (there is no CPU path)")
        shape = x1.shape
        x1c, x2c, gc = (t.contiguous().view(-1, D) for t in (x1, x2, g.to(x1.dtype)))
        rows = x1c.shape[0]
        xw = None
        if x_weights_after_norm is not None:
            xw = x_weights_after_norm.contiguous().view(-1, 2)
            if xw.dtype not in (torch.bfloat16, torch.float32):
                xw = xw.float()
            assert xw.shape[0] == rows
        w1, w2 = self.weight1, self.weight2
        if w1 is not None and w1.dtype not in (torch.bfloat16, torch.float32):
            w1, w2 = w1.float(), w2.float()
        y = _NormGateMix.apply(x1c, x2c, gc, xw, w1, w2, float(self.eps), 1 if self.activation == 'sigmoid' else 0)
        return y.view(shape)
