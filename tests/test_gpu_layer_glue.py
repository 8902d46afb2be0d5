"""GPU tests (-m gpu) of the bandwidth kernels around the hybrid attention op (short convolution + SiLU, RMSNorm with
the fused residual add, SwiGLU, block mean), forward and backward, against the same expressions evaluated by PyTorch
in float64 on the CPU from the same bf16 inputs."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
TOL = 1e-2


def close(got, ref, what, tol=TOL):
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), what
    s = max(1.0, float(ref.abs().max()) * 0.1)
    err = (got - ref).abs()
    assert bool((err <= tol * ref.abs() + tol * s).all()), f"{what}: max err {err.max().item():.4g} (ref max {ref.abs().max().item():.4g})"


@pytest.mark.parametrize("B,T,D,bias,act", [(2, 100, 64, False, "silu"), (1, 1000, 1024, False, "silu"), (2, 77, 128, True, "silu"),
                                            (1, 300, 256, False, None), (3, 3, 64, False, "silu"), (1, 130, 72, True, "silu"),
                                            (2, 64, 136, False, "silu")])
def test_short_conv(B, T, D, bias, act):
    from neuralattentionsearchlinear_b200.modules import ShortConvolution
    torch.manual_seed(T + D)
    conv = ShortConvolution(D, 4, bias=bias, activation=act).cuda().bfloat16()
    x = torch.randn(B, T, D).bfloat16()
    dy = torch.randn(B, T, D).bfloat16()
    xg = x.cuda().requires_grad_(True)
    y, _ = conv(xg)
    (y.float() * dy.cuda().float()).sum().backward()
    xr = x.double().requires_grad_(True)
    w = conv.weight.detach().double().cpu().requires_grad_(True)
    b = conv.bias.detach().double().cpu().requires_grad_(True) if bias else None
    pre = F.conv1d(xr.transpose(1, 2), w, b, padding=3, groups=D)[..., :T]
    yr = (F.silu(pre) if act else pre).transpose(1, 2)
    (yr * dy.double()).sum().backward()
    close(y, yr, "y")
    close(xg.grad, xr.grad, "dx")
    close(conv.weight.grad, w.grad, "dw")
    if bias:
        close(conv.bias.grad, b.grad, "dbias")


@pytest.mark.parametrize("D,rows_shape,with_res", [(64, (2, 50, 4), False), (128, (3, 33, 2), False), (1024, (2, 70), True),
                                                   (2048, (1, 40), True), (256, (5, 7), False), (512, (4, 9), True), (128, (3, 5), True),
                                                   (256, (1, 3), True), (64, (1, 1), False)])
def test_rmsnorm(D, rows_shape, with_res):
    from neuralattentionsearchlinear_b200.modules import RMSNorm
    torch.manual_seed(D)
    norm = RMSNorm(D, eps=1e-6).cuda().bfloat16()
    with torch.no_grad():
        norm.weight.copy_(1 + 0.2 * torch.randn(D))
    x = torch.randn(*rows_shape, D).bfloat16()
    r = torch.randn(*rows_shape, D).bfloat16() if with_res else None
    dy = torch.randn(*rows_shape, D).bfloat16()
    ds = torch.randn(*rows_shape, D).bfloat16()
    xg = x.cuda().requires_grad_(True)
    rg = r.cuda().requires_grad_(True) if with_res else None
    if with_res:
        y, s = norm(xg, rg, True)
        ((y.float() * dy.cuda().float()).sum() + (s.float() * ds.cuda().float()).sum()).backward()
    else:
        y = norm(xg)
        (y.float() * dy.cuda().float()).sum().backward()
    xr = x.double().requires_grad_(True)
    rr = r.double().requires_grad_(True) if with_res else None
    w = norm.weight.detach().double().cpu().requires_grad_(True)
    sr = xr + rr if with_res else xr
    if with_res:
        # the residual stream is stored in bf16 and the stored value is what gets normalised
        sr = sr + (sr.detach().bfloat16().double() - sr.detach())
    yr = sr * torch.rsqrt(sr.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    loss = (yr * dy.double()).sum() + ((sr * ds.double()).sum() if with_res else 0.0)
    loss.backward()
    close(y, yr, "y")
    close(xg.grad, xr.grad, "dx")
    close(norm.weight.grad, w.grad, "dw")
    if with_res:
        close(s, sr, "x + residual")
        close(rg.grad, rr.grad, "dresidual")


def test_swiglu_and_block_mean():
    from neuralattentionsearchlinear_b200.modules import mean_pooling, swiglu
    torch.manual_seed(0)
    a, b, dy = (torch.randn(3, 50, 2816).bfloat16() for _ in range(3))
    ag, bg = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    y = swiglu(ag, bg)
    (y.float() * dy.cuda().float()).sum().backward()
    ar, br = a.double().requires_grad_(True), b.double().requires_grad_(True)
    yr = F.silu(ar) * br
    (yr * dy.double()).sum().backward()
    close(y, yr, "swiglu")
    close(ag.grad, ar.grad, "da")
    close(bg.grad, br.grad, "db")
    x = torch.randn(2, 300, 1, 256).bfloat16()
    dyp = torch.randn(2, 5, 1, 256).bfloat16()
    xg = x.cuda().requires_grad_(True)
    p = mean_pooling(xg, 64)
    (p.float() * dyp.cuda().float()).sum().backward()
    xr = x.double().requires_grad_(True)
    pr = torch.stack([xr[:, i * 64:(i + 1) * 64].mean(1) for i in range(5)], 1)
    (pr * dyp.double()).sum().backward()
    close(p, pr, "block mean")
    close(xg.grad, xr.grad, "d(block mean)")


def test_short_conv_with_cache_is_bit_identical_to_one_pass():
    """Decoding feeds the convolution piece by piece with the cached tail; every output must equal the one-pass output bit
    for bit (the linear branch's q, k, v are then the same in both, whatever the conditioning of what follows)."""
    from neuralattentionsearchlinear_b200.modules import ShortConvolution
    torch.manual_seed(5)
    conv = ShortConvolution(256, 4, bias=False, activation='silu').cuda().bfloat16()
    x = torch.randn(2, 150, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        full, fin = conv(x, output_final_state=True)
        outs, state, t = [], None, 0
        for n in (70, 1, 1, 5, 2, 64, 7):
            y, state = conv(x[:, t:t + n], cache=state, output_final_state=True)
            outs.append(y)
            t += n
    assert t == 150
    assert torch.equal(torch.cat(outs, 1), full)
    assert torch.equal(state, fin)
