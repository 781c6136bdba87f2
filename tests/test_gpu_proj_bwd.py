"""Backward pass of the block-diagonal projection (lffn_proj_bwd) against fp64 autograd over the reference's own
formulation: per rotation and stage torch.einsum("bni,noi->bno") then a product with the Sylvester matrix
(bh4/kernel.py:23-36), then 0.7 * P + 0.3 * tile(x_pad), slice, + bias (lookup.py:29-39).  Bar: gradients within
1e-3 relative (the fp32 bound of the task); measured agreement is about 1e-6.  The kernels use no atomics, so two
runs must give the same bits."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from lookupffn_b200 import _lib

    _lib.lib()
    return torch.device("cuda:0")


def rel(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def reference_fp64(x, weight, bias, out_dim, had_scale, mix_a, mix_b):
    N, d_in = x.shape
    R, S, NB, BS, _ = weight.shape
    D = NB * BS
    H = torch.ones(1, 1, dtype=torch.float64, device=x.device)
    while H.shape[0] < D:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    up = torch.nn.functional.pad(x, (0, D - d_in))
    outs = []
    for r in range(R):
        y = up
        for s in range(S):
            y = torch.einsum("bni,noi->bno", y.reshape(N, NB, BS), weight[r, s]).reshape(N, D)
            y = (y @ H) * had_scale
        outs.append(y)
    z = mix_a * torch.cat(outs, -1) + mix_b * up.repeat(1, R)
    return z[:, :out_dim] + bias


CASES = [
    # N, d_in, D, S, out_dim, had_scale, (mix_a, mix_b)
    (100, 512, 512, 4, 1024, 1.0, (0.7, 0.3)),          # the reference layer: t128, 8 bits, hidden 512
    (77, 200, 256, 4, 600, 1.0, (0.7, 0.3)),            # padded input, ragged tile, out_dim not a multiple of D
    (300, 768, 1024, 4, 2048, 1.0 / 32, (1.0, 0.0)),    # D = 1024: the narrow tile pipeline, normalised transform
    (64, 512, 512, 2, 512, 1.0, (0.7, 0.3)),            # two stages, one rotation
    (1, 256, 256, 4, 256, 1.0, (0.7, 0.3)),             # a single token
    (9491, 512, 512, 4, 1024, 1.0, (0.7, 0.3)),         # two or three tiles per CTA: the prefetched gradient tiles, ragged end
]


@pytest.mark.parametrize("case", CASES, ids=[f"p{i}" for i in range(len(CASES))])
def test_proj_bwd_matches_fp64_autograd(dev, case):
    from lookupffn_b200 import ops

    N, d_in, D, S, out_dim, hs, (mix_a, mix_b) = case
    R = max(1, -(-out_dim // D))
    g = torch.Generator(device=dev).manual_seed(N + D)
    x = torch.randn(N, d_in, generator=g, device=dev)
    # of order one through the stages whatever had_scale is
    weight = torch.randn(R, S, D // 64, 64, 64, generator=g, device=dev) / (np.sqrt(64.0) * (np.sqrt(D) * hs if hs != 1.0 else np.sqrt(D)))
    bias = 0.05 * torch.randn(out_dim, generator=g, device=dev)
    dz = torch.randn(N, out_dim, generator=g, device=dev)
    wt = weight.transpose(-1, -2).contiguous()
    du, dw, db = ops.proj_bwd(x, weight, wt, out_dim, dz, hs, mix_a, mix_b)
    du2, dw2, db2 = ops.proj_bwd(x, weight, wt, out_dim, dz, hs, mix_a, mix_b)
    assert torch.equal(du, du2) and torch.equal(dw, dw2) and torch.equal(db, db2)
    # the training forward keeps the stage inputs: same z as the plain kernel, same gradients as recomputing
    z_t, acts = ops.proj_fwd_train(x, wt, bias, out_dim, hs, mix_a, mix_b)
    desc = ops.make_hash_desc(d_in, wt, bias, out_dim, 1, transpose_w=True, had_scale=hs, mix_a=mix_a, mix_b=mix_b,
                              weight_mode=ops.WEIGHT_ONES)
    assert torch.equal(z_t, ops.hash_fwd(x, desc, want_z=True, want_codes=False)[2])
    du3, dw3, db3 = ops.proj_bwd(x, weight, wt, out_dim, dz, hs, mix_a, mix_b, acts=acts)
    assert torch.equal(du, du3) and torch.equal(dw, dw3) and torch.equal(db, db3)

    x64 = x.double().requires_grad_(True)
    w64 = weight.double().requires_grad_(True)
    b64 = bias.double().requires_grad_(True)
    z = reference_fp64(x64, w64, b64, out_dim, float(np.float32(hs)), float(np.float32(mix_a)), float(np.float32(mix_b)))
    z.backward(dz.double())
    assert rel(du[:, :d_in], x64.grad) < 1e-4
    if d_in < D:  # the padded columns receive a gradient too; nothing reads it
        assert torch.isfinite(du).all()
    assert rel(dw, w64.grad) < 1e-4
    assert rel(db, b64.grad) < 1e-5
    from lookupffn_b200 import _lib as L

    assert L.device_status(dev) == 0


def test_projection_autograd_function_uses_the_kernels(dev):
    """ops.Projection (what Hashing.forward runs in training) end to end: forward z and all three gradients against
    fp64 autograd, with partial requires_grad combinations."""
    from lookupffn_b200 import ops
    from lookupffn_b200.lookup import BH4

    torch.manual_seed(0)
    mod = BH4(500, 1500, 64).to(dev)
    with torch.no_grad():
        mod.bias.normal_(0, 0.05)
    x = torch.randn(90, 500, device=dev, requires_grad=True)
    wk, tw = mod.kernel_weight()
    z = ops.Projection.apply(x, mod.weight, mod.bias, mod.had_scale, mod.mix[0], mod.mix[1], wk, tw)
    dz = torch.randn_like(z)
    z.backward(dz)
    x64 = x.detach().double().requires_grad_(True)
    w64 = mod.weight.detach().double().requires_grad_(True)
    b64 = mod.bias.detach().double().requires_grad_(True)
    z64 = reference_fp64(x64, w64, b64, 1500, 1.0, float(np.float32(0.7)), float(np.float32(1 - 0.7)))
    z64.backward(dz.double())
    assert rel(z.detach(), z64.detach()) < 1e-5
    assert rel(x.grad, x64.grad) < 1e-4 and rel(mod.weight.grad, w64.grad) < 1e-4 and rel(mod.bias.grad, b64.grad) < 1e-5
    # only the input needs a gradient (frozen projection)
    mod.weight.requires_grad_(False)
    mod.bias.requires_grad_(False)
    x3 = x.detach().clone().requires_grad_(True)
    ops.Projection.apply(x3, mod.weight, mod.bias, mod.had_scale, mod.mix[0], mod.mix[1], wk, tw).backward(dz)
    assert torch.equal(x3.grad, x.grad)


@pytest.mark.parametrize("d", [256, 512, 768, 1024])
def test_layernorm_backward_matches_fp64_autograd(d):
    """lffn_layernorm_bwd against torch autograd in fp64 (1e-5 of each gradient's largest value), on a ragged row
    count, and bit-identical when run twice (fixed summation order)."""
    from lookupffn_b200 import ops

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(d)
    N = 4099
    x = torch.randn(N, d, generator=g, device=dev) * 1.7 + 0.3
    du = torch.randn(N, d, generator=g, device=dev)
    gamma = torch.rand(d, generator=g, device=dev) + 0.5
    beta = torch.randn(d, generator=g, device=dev)
    x64 = x.double().requires_grad_(True)
    g64, b64 = gamma.double().requires_grad_(True), beta.double().requires_grad_(True)
    torch.nn.functional.layer_norm(x64, (d,), g64, b64, 1e-5).backward(du.double())
    dx, dgamma, dbeta = ops.layernorm_bwd(x, du, gamma, 1e-5)
    for got, want in ((dx, x64.grad), (dgamma, g64.grad), (dbeta, b64.grad)):
        assert float((got.double() - want).abs().max() / want.abs().max()) < 1e-5
    dx2, dgamma2, dbeta2 = ops.layernorm_bwd(x, du, gamma, 1e-5)
    assert torch.equal(dx, dx2) and torch.equal(dgamma, dgamma2) and torch.equal(dbeta, dbeta2)


def test_layer_norm_function_routes_training_through_the_kernel():
    from lookupffn_b200 import ops

    dev = torch.device("cuda:0")
    ln = torch.nn.LayerNorm(512, eps=1e-5).to(dev)
    with torch.no_grad():
        ln.weight.uniform_(0.5, 1.5)
        ln.bias.normal_()
    x = torch.randn(3, 77, 512, device=dev, requires_grad=True)
    y = ops.layer_norm(x, ln)
    assert y.grad_fn is not None and "LayerNormFn" in type(y.grad_fn).__name__
    y.square().sum().backward()
    got = (x.grad.clone(), ln.weight.grad.clone(), ln.bias.grad.clone())
    x.grad = None
    ln.zero_grad()
    ln(x).square().sum().backward()
    for a, b in zip(got, (x.grad, ln.weight.grad, ln.bias.grad)):
        assert float((a - b).abs().max() / b.abs().max()) < 1e-5
    with torch.no_grad():
        assert ops.layer_norm(x, ln).grad_fn is None  # inference: torch's module


def test_bias_gradient_is_the_column_sum_and_rides_through_the_gather_function():
    from lookupffn_b200 import ops

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(3)
    dy = torch.randn(5001, 768, generator=g, device=dev)
    got = ops.bias_grad(dy)
    want = dy.double().sum(0)
    assert float((got.double() - want).abs().max() / want.abs().max()) < 1e-6
    assert torch.equal(got, ops.bias_grad(dy))  # fixed summation order
    # through the autograd function: forward adds the bias in the kernel, backward returns its gradient
    S, d, N, I = 300, 64, 257, 7
    tables = torch.randn(S, d, generator=g, device=dev, requires_grad=True)
    bias = torch.randn(d, generator=g, device=dev, requires_grad=True)
    idx = torch.randint(0, S, (N, I), generator=g, device=dev, dtype=torch.int32)
    w = torch.randn(N, I, generator=g, device=dev, requires_grad=True)
    out = ops.gather(idx, w, tables, training=True, bias=bias)
    ref = (tables[idx.long()] * w[..., None]).sum(1) + bias
    assert float((out - ref).detach().abs().max() / ref.detach().abs().max()) < 1e-5
    gy = torch.randn(N, d, generator=g, device=dev)
    out.backward(gy)
    gb, gw, gt = bias.grad.clone(), w.grad.clone(), tables.grad.clone()
    bias.grad = w.grad = tables.grad = None
    ref.backward(gy)
    for a, b in ((gb, bias.grad), (gw, w.grad), (gt, tables.grad)):
        assert float((a - b).abs().max() / b.abs().max()) < 1e-5
