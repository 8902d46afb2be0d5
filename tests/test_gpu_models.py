"""GPU tests (-m gpu) of the decoder model around the NAtSL-GDN layer: it trains (every parameter receives a finite
gradient), and the gradients of a two-layer slice equal those of a CPU restatement in which the hybrid attention op is
the oracle (fp32, autograd through the chunk form and the masked softmax; the reference's ``dnats`` injected as the
gradient of the block types, since it is not a derivative of the forward)."""
import copy
import functools

import pytest
import torch

from oracle import attn as oattn
from oracle import gdn as ogdn
from oracle import grad as ograd

pytestmark = pytest.mark.gpu


def _small_config(**over):
    from neuralattentionsearchlinear_b200.models import NeuralAttentionSearchLineraAttnGDNConfig
    kw = dict(hidden_size=256, expand_v=1.0, head_dim=64, num_heads=4, num_attn_heads=4, num_hidden_layers=2,
              vocab_size=512, nats_block_size=64, ops_for_incomplete_chunks='all', attn_apply_pos_encoding=False,
              attn_qk_norm=True, attn_with_short_conv=True, decay_for_non_gdn_blocks=True, norm_eps=1e-6)
    kw.update(over)
    return NeuralAttentionSearchLineraAttnGDNConfig(**kw)


def test_model_trains_every_parameter():
    from neuralattentionsearchlinear_b200.models import NeuralAttentionSearchLinearAttnGDNForCausalLM
    torch.manual_seed(0)
    model = NeuralAttentionSearchLinearAttnGDNForCausalLM(_small_config(head_dim=128, num_heads=2, num_attn_heads=4)).cuda().bfloat16()
    model.train()
    ids = torch.randint(0, 512, (2, 256), device="cuda")
    out = model(input_ids=ids, labels=ids)
    assert out["logits"] is None and torch.isfinite(out["loss"])
    out["loss"].backward()
    for name, p in model.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), name
        assert float(p.grad.float().abs().max()) > 0, f"{name} received a zero gradient"
    model.eval()
    with torch.no_grad():
        ev = model(input_ids=ids, labels=ids)
    assert ev["logits"].shape == (2, 256, 512)
    assert abs(float(ev["loss"]) - float(out["loss"])) < 5e-2       # train op and chunk-inference op agree


class _Tap(torch.autograd.Function):
    """Identity on (o_lin, o_attn) whose backward also hands the block types the reference's ``dnats``."""

    @staticmethod
    def forward(ctx, o_l, o_a, types, payload):
        ctx.payload = payload
        return o_l.clone(), o_a.clone()

    @staticmethod
    def backward(ctx, do_l, do_a):
        p = ctx.payload
        with torch.enable_grad():
            dn_a = ograd.attn_grads(p["q_attn"], p["k_attn"], p["v_attn"], p["sel"][..., 0], do_a, nbs=64,
                                    own_chunk=True)["dnats"]
            dn_l = ograd.dnats_linear(p["q"], p["k"], p["v"], p["g"], p["beta"], p["sel"][..., 1], do_l, None,
                                      invalid_blocks=p["invalid"], decay=p["decay"])
        return do_l, do_a, torch.stack([dn_a, dn_l], -1), None


def _ref_layer_forward(layer, types_dev, hidden_states, **kwargs):
    """The layer on the CPU: its own projections, the oracle as the hybrid attention op, the mixing formula."""
    layer.nats_sample_func = lambda lg: types_dev - lg.softmax(-1).detach() + lg.softmax(-1)   # the device's decisions
    p = layer.project(hidden_states)
    sel = p["types"].detach()
    T = hidden_states.shape[1]
    o_l, _ = ogdn.linear_chunk(p["q"], p["k"], p["v"], p["g"], p["beta"], sel[..., 1], nbs=64,
                               decay=layer.decay_for_non_gdn_blocks, use_l2norm=True)
    mask = oattn.attn_mask(sel[..., 0], T, 64, layer.num_attn_heads)
    o_a, _ = oattn.attn_sdpa(p["q_attn"], p["k_attn"], p["v_attn"], mask)
    det = lambda x: x.detach()
    payload = dict(q=det(p["q"]), k=det(p["k"]), v=det(p["v"]), g=det(p["g"]), beta=det(p["beta"]), sel=sel,
                   q_attn=det(p["q_attn"]), k_attn=det(p["k_attn"]), v_attn=det(p["v_attn"]),
                   invalid=layer.compute_dnats_for_invalid_blocks_linear_att, decay=layer.decay_for_non_gdn_blocks)
    o_l, o_a = _Tap.apply(o_l, o_a, p["types"], payload)
    g = layer.g_proj(hidden_states).unflatten(-1, (-1, layer.head_v_dim)).reshape(o_a.shape)
    rms = lambda x: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + layer.o_norm.eps)
    w = p["o_weights"]
    o = (rms(o_l.reshape(o_a.shape)) * layer.o_norm.weight1 * w[..., :1] + rms(o_a) * layer.o_norm.weight2 * w[..., 1:])
    o = o * g * torch.sigmoid(g)
    return layer.o_proj(o.flatten(-2)), None, None


def test_two_layer_gradients_against_oracle():
    from neuralattentionsearchlinear_b200.models import NeuralAttentionSearchLinearAttnGDNForCausalLM
    torch.manual_seed(1)
    cfg = _small_config()
    model = NeuralAttentionSearchLinearAttnGDNForCausalLM(cfg).bfloat16()
    ref = copy.deepcopy(model).float()                     # same bf16-rounded weights, fp32 arithmetic, on the CPU
    model = model.cuda().train()
    ref.train()
    ids = torch.randint(0, cfg.vocab_size, (2, 256))
    # record the device's 0/1 decisions (discrete: a bf16 near-tie must not send the two runs down different paths)
    decisions = []
    for layer in model.model.layers:
        orig = layer.attn.nats_sample_func
        layer.attn.nats_sample_func = (lambda f: lambda lg: decisions.append(f(lg).detach().float().cpu()) or f(lg))(orig)
    out = model(input_ids=ids.cuda(), labels=ids.cuda())
    out["loss"].backward()
    assert len(decisions) == 2
    for layer, dec in zip(ref.model.layers, decisions):
        layer.attn.forward = functools.partial(_ref_layer_forward, layer.attn, dec)
    ref_out = ref(input_ids=ids, labels=ids)
    ref_out["loss"].backward()
    assert abs(float(out["loss"]) - float(ref_out["loss"])) < 2e-2 * max(1.0, abs(float(ref_out["loss"])))
    worst = []
    for (name, p), (_, r) in zip(model.named_parameters(), ref.named_parameters()):
        got, want = p.grad.float().cpu().flatten(), r.grad.float().flatten()
        assert torch.isfinite(got).all(), name
        rel = float((got - want).norm() / want.norm().clamp_min(1e-12))
        cos = float(torch.dot(got, want) / (got.norm() * want.norm()).clamp_min(1e-20))
        worst.append((rel, cos, name))
        # bf16 activations through two blocks and the LM head: a few per cent of noise per parameter tensor
        assert cos > 0.99 and rel < 0.15, f"{name}: relative L2 error {rel:.3f}, cosine {cos:.4f}"
    print("largest relative errors:", sorted(worst, reverse=True)[:5])


def test_fused_cross_entropy_rows_match_torch():
    """The loss head (slice-wise logits -> loss and gradients, one kernel per slice for the softmax part) against
    torch's cross entropy with autograd in fp32 on the same bf16 operands; ignored labels, a ragged last slice."""
    from neuralattentionsearchlinear_b200.models import _ChunkedLinearCrossEntropy
    torch.manual_seed(3)
    n, hdim, vocab = 1000, 256, 4096
    hidden = (torch.randn(n, hdim) * 0.5).bfloat16().cuda().requires_grad_(True)
    weight = (torch.randn(vocab, hdim) * 0.05).bfloat16().cuda().requires_grad_(True)
    labels = torch.randint(0, vocab, (n,)).cuda()
    labels[::7] = -100
    loss = _ChunkedLinearCrossEntropy.apply(hidden, weight, labels, -100, 384)
    loss.backward()
    h32 = hidden.detach().float().requires_grad_(True)
    w32 = weight.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy((h32 @ w32.t()).bfloat16().float(), labels, ignore_index=-100)
    # the straight-through of the bf16 rounding of the logits: differentiate the unrounded expression
    ref_g = torch.nn.functional.cross_entropy(h32 @ w32.t(), labels, ignore_index=-100)
    ref_g.backward()
    assert abs(float(loss) - float(ref)) < 2e-3 * max(1.0, abs(float(ref)))
    for got, want, what in ((hidden.grad, h32.grad, "d hidden"), (weight.grad, w32.grad, "d weight")):
        err = (got.float() - want).abs().max().item()
        assert err <= 2e-2 * want.abs().max().item() + 1e-6, (what, err, want.abs().max().item())
