"""The benchmark configurations that are parity cases rather than bench lines:
configuration 1 (MXFP8 Linear forward, 4096^3, against the oracle: codes and scales bit-exact,
Y within tolerance) and a small instance of configuration 5 (Llama-style decoder block stack
with every Linear swapped for the drop-in module under the MXFP8 recipe, one forward+backward
step) against the same model in bf16."""
import math

import numpy as np
import pytest
import torch

from helpers import mismatch, np_u8, seeded_bf16
from minitransformer_b200 import kernels as K
from minitransformer_b200.module import config
from minitransformer_b200.module.linear import Linear
from oracle import gemm, mxfp8

pytestmark = pytest.mark.gpu


def test_config1_mxfp8_linear_forward_4096():
    """X [4096,4096] ~ N(0,1), W [4096,4096] ~ N(0,0.02), 1x32 blocks along K, E8M0 scales."""
    n = 4096
    tx, x = seeded_bf16((n, n), 1234, 1.0)
    tw, w = seeded_bf16((n, n), 1235, 0.02)
    ox, ow = mxfp8.quantize(x, return_transpose=False), mxfp8.quantize(w, return_transpose=False)
    params = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
    op = params.quantize_op
    qx = op.quantize(tx.cuda(), params.x_params)
    qw = op.quantize(tw.cuda(), params.w_params)
    assert mismatch(np_u8(qx.data), ox["data"]) == 0 and mismatch(np_u8(qx.scale), ox["scale"]) == 0
    assert mismatch(np_u8(qw.data), ow["data"]) == 0 and mismatch(np_u8(qw.scale), ow["scale"]) == 0
    lin = Linear(n, n, bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params)
    with torch.no_grad():
        lin.weight.copy_(tw)
        y = lin(tx.cuda())
    ref = gemm.qgemm_mxfp8(ox["data"], ox["scale"], ow["data"], ow["scale"], fused=True)
    assert gemm.rel_frobenius(y.float().cpu().numpy(), ref) <= 1e-3
    assert K.read_device_status() == 0


class _RMSNorm(torch.nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(dim, dtype=torch.bfloat16, device="cuda"))

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)).to(x.dtype) * self.weight


class _Block(torch.nn.Module):
    def __init__(self, hidden, heads, kv_heads, ffn, params):
        super().__init__()
        self.heads, self.kv_heads, self.hd = heads, kv_heads, hidden // heads
        kw = dict(bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params,
                  init_method=lambda t: torch.nn.init.normal_(t, std=0.02))
        self.norm1, self.norm2 = _RMSNorm(hidden), _RMSNorm(hidden)
        self.qkv = Linear(hidden, (heads + 2 * kv_heads) * self.hd, **kw)
        self.proj = Linear(hidden, hidden, **kw)
        self.fc1 = Linear(hidden, 2 * ffn, **kw)      # gated: [gate | up]
        self.fc2 = Linear(ffn, hidden, **kw)

    def forward(self, x):                             # x [B, S, H]
        B, S, H = x.shape
        qkv = self.qkv(self.norm1(x))
        q, k, v = qkv.split([self.heads * self.hd, self.kv_heads * self.hd, self.kv_heads * self.hd], dim=-1)
        q = q.view(B, S, self.heads, self.hd).transpose(1, 2)
        k = k.view(B, S, self.kv_heads, self.hd).transpose(1, 2).repeat_interleave(self.heads // self.kv_heads, 1)
        v = v.view(B, S, self.kv_heads, self.hd).transpose(1, 2).repeat_interleave(self.heads // self.kv_heads, 1)
        a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, S, H))
        g, u = self.fc1(self.norm2(x)).chunk(2, dim=-1)
        return x + self.fc2(torch.nn.functional.silu(g) * u)


class _Decoder(torch.nn.Module):
    def __init__(self, layers, hidden, heads, kv_heads, ffn, vocab, params):
        super().__init__()
        self.emb = torch.nn.Embedding(vocab, hidden, dtype=torch.bfloat16, device="cuda")
        self.blocks = torch.nn.ModuleList([_Block(hidden, heads, kv_heads, ffn, params) for _ in range(layers)])
        self.norm = _RMSNorm(hidden)
        self.head = Linear(hidden, vocab, bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params,
                           init_method=lambda t: torch.nn.init.normal_(t, std=0.02))

    def forward(self, ids):
        x = self.emb(ids)
        for b in self.blocks:
            x = b(x)
        return self.head(self.norm(x))


def test_config5_small_llama_style_step_mxfp8_vs_bf16():
    """Scaled-down instance of the 8-layer decoder configuration (2 layers, hidden 256, 4 heads /
    2 KV heads, gated ffn 512, vocab 512, seq 128 x micro-batch 2, random-init N(0,0.02) weights,
    uniform token ids, torch SDPA): one forward+backward with every Linear under the MXFP8
    recipe stays within quantization noise of the bf16 model with the same weights."""
    torch.manual_seed(0)
    dims = dict(layers=2, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=512)
    qp = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
    bp = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.NON_QUANTIZE)
    mq, mb = _Decoder(params=qp, **dims), _Decoder(params=bp, **dims)
    mb.load_state_dict(mq.state_dict())
    ids = torch.randint(0, dims["vocab"], (2, 128), device="cuda")
    tgt = torch.randint(0, dims["vocab"], (2, 128), device="cuda")
    losses, grads = [], []
    for m in (mq, mb):
        logits = m(ids)
        loss = torch.nn.functional.cross_entropy(logits.float().view(-1, dims["vocab"]), tgt.view(-1))
        loss.backward()
        losses.append(loss.item())
        grads.append(torch.cat([p.grad.float().flatten() for n, p in sorted(m.named_parameters()) if p.grad is not None]))
    assert math.isfinite(losses[0]) and abs(losses[0] - losses[1]) / losses[1] < 0.02, losses
    cos = float(torch.nn.functional.cosine_similarity(grads[0], grads[1], dim=0))
    assert cos > 0.97, cos
    assert K.read_device_status() == 0


def _check_linear_slices(name, x, w, dy, y, dx, dw):
    """One Linear of the decoder at size against the MXFP8 oracle, on slices small enough for
    numpy: y on a token x feature block (row-wise copies of x and w), dx on a token x input
    block (row-wise dy, transposed copy of w), dw on a feature x input block (transposed copies
    of dy and x over ALL tokens). Blocks of the transposed copies run along the sliced-away
    dimension, so quantizing the slice gives exactly the rows of the full copy."""
    f32 = lambda t: t.detach().float().cpu().numpy()
    T, Kd = x.shape
    N = w.shape[0]
    r0, n0, k0 = T // 2 - 64, min(N - 128, 3 * 128), Kd // 2
    rs, ns, ks = slice(r0, r0 + 128), slice(n0, n0 + 128), slice(k0, k0 + 128)
    qx = mxfp8.quantize(f32(x[rs]), return_transpose=False)
    qw = mxfp8.quantize(f32(w[ns]), return_transpose=False)
    ref_y = gemm.qgemm_mxfp8(qx["data"], qx["scale"], qw["data"], qw["scale"], fused=True)
    assert gemm.rel_frobenius(f32(y[rs, ns]), ref_y) <= 1e-3, (name, "y")
    qg = mxfp8.quantize(f32(dy[rs]), return_transpose=False)
    qwt = mxfp8.quantize(f32(w[:, ks]), return_transpose=True)
    ref_dx = gemm.qgemm_mxfp8(qg["data"], qg["scale"], qwt["data_t"], qwt["scale_t"], fused=True)
    assert gemm.rel_frobenius(f32(dx[rs, ks]), ref_dx) <= 1e-3, (name, "dx")
    qgt = mxfp8.quantize(f32(dy[:, ns]), return_transpose=True)
    qxt = mxfp8.quantize(f32(x[:, ks]), return_transpose=True)
    ref_dw = gemm.qgemm_mxfp8(qgt["data_t"], qgt["scale_t"], qxt["data_t"], qxt["scale_t"], out_bf16=True, fused=True)
    assert gemm.rel_frobenius(f32(dw[ns, ks]), ref_dw) <= 1e-3, (name, "dw")


def test_config5_one_layer_at_size_every_linear_against_oracle():
    """One decoder layer of configuration 5 at full width (hidden 4096, 32 heads / 8 KV heads,
    gated ffn 14336, seq 4096 x micro-batch 2 = 8192 tokens, MXFP8 recipe): the inputs and
    gradients each of the four Linears saw in the step are captured with hooks and every Linear's
    output, input gradient and weight gradient are compared with the oracle on slices."""
    torch.manual_seed(1)
    qp = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
    blk = _Block(4096, 32, 8, 14336, qp)
    seen = {}

    def watch(name, mod):
        def hook(m, inp, out):
            rec = seen.setdefault(name, {})
            rec["x"], rec["y"] = inp[0].detach(), out.detach()
            inp[0].register_hook(lambda g: rec.__setitem__("dx", g.detach()))
            out.register_hook(lambda g: rec.__setitem__("dy", g.detach()))
        mod.register_forward_hook(hook)

    for name in ("qkv", "proj", "fc1", "fc2"):
        watch(name, getattr(blk, name))
    x = torch.randn(2, 4096, 4096, device="cuda").to(torch.bfloat16).requires_grad_(True)
    out = blk(x)
    out.backward((torch.randn_like(out.float()) * 1e-3).to(torch.bfloat16))
    torch.cuda.synchronize()
    for name in ("qkv", "proj", "fc1", "fc2"):
        rec, lin = seen[name], getattr(blk, name)
        flat = lambda t: t.reshape(-1, t.shape[-1])
        _check_linear_slices(name, flat(rec["x"]), lin.weight.detach(), flat(rec["dy"]), flat(rec["y"]),
                             flat(rec["dx"]), lin.weight.grad)
    assert K.read_device_status() == 0
