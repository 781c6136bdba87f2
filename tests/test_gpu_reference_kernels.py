"""The library's kernels against the reference's own CUDA kernels, both running on the GPU.

oracle/_ref holds the reference's CUDA extensions compiled unmodified for sm_100a (oracle/build.py):
`gather_add` (gather/cuda/extension/*: weighted_vector_gather_add / indexed_inner_product /
weighted_vector_scatter_add, fp32 and fp16) and `fast_hadamard_transform_kernel`
(bh4/fast_hadamard_transform/extension/*).  Inputs stay inside what those kernels accept (contiguous, even list
length, vector_dim a multiple of 64, valid indices, one token per CTA).

Tolerances: fp32 gather and the fp32 Hadamard transform are bit-exact (same operation order, one rounding per
step); the inner product and the atomics-based scatter differ in summation order (1e-5 / 1e-4 of the largest
value); the reference's fp16 kernels accumulate in fp16, ours store bf16 and accumulate in fp32 (2e-2).
"""
import numpy as np
import pytest
import torch

from oracle import build as obuild

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def ref_gather(dev):
    mod = obuild.load_ref_module("gather_add")
    if mod is None:
        pytest.skip("oracle/_ref/gather_add not built (python oracle/build.py with the reference tree present)")
    return mod


@pytest.fixture(scope="module")
def ref_fht(dev):
    mod = obuild.load_ref_module("fast_hadamard_transform_kernel")
    if mod is None:
        pytest.skip("oracle/_ref/fast_hadamard_transform_kernel not built")
    return mod


def make_case(dev, N, I, S, d, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    idx = torch.randint(0, S, (N, I), generator=g, device=dev, dtype=torch.int32)
    w = torch.rand(N, I, generator=g, device=dev)
    src = 0.02 * torch.randn(S, d, generator=g, device=dev)
    dy = torch.randn(N, d, generator=g, device=dev)
    return idx, w, src, dy


CASES = [(257, 64, 4096, 512), (100, 256, 65536, 768), (64, 30, 1000, 64), (33, 512, 131072, 1024)]


@pytest.mark.parametrize("case", CASES, ids=[f"g{i}" for i in range(len(CASES))])
def test_gather_fp32_bit_exact_against_reference_kernel(dev, ref_gather, case):
    from lookupffn_b200 import ops

    N, I, S, d = case
    idx, w, src, _ = make_case(dev, N, I, S, d, seed=N + I)
    ref = torch.zeros(N, d, device=dev)
    ref_gather.weighted_vector_gather_add_fp32(idx, src, w, ref)
    out = ops.weighted_vector_gather_add(idx, src, w)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


@pytest.mark.parametrize("case", CASES[:3], ids=[f"g{i}" for i in range(3)])
def test_gather_16bit_against_reference_fp16_kernel(dev, ref_gather, case):
    from lookupffn_b200 import ops

    N, I, S, d = case
    idx, w, src, _ = make_case(dev, N, I, S, d, seed=7 * N + I)
    ref = torch.zeros(N, d, device=dev, dtype=torch.float16)
    ref_gather.weighted_vector_gather_add_fp16(idx, src.half().contiguous(), w.half().contiguous(), ref)
    out = ops.weighted_vector_gather_add(idx, src.to(torch.bfloat16), w)
    exact = ops.weighted_vector_gather_add(idx, src, w)
    torch.cuda.synchronize()
    assert rel_err(out.float().cpu(), exact.cpu()) < 2e-2
    assert rel_err(ref.float().cpu(), exact.cpu()) < 2e-2          # the reference kernel under the same bound
    assert rel_err(out.float().cpu(), ref.float().cpu()) < 2e-2


@pytest.mark.parametrize("case", CASES, ids=[f"g{i}" for i in range(len(CASES))])
def test_backward_kernels_against_reference_kernels(dev, ref_gather, case):
    from lookupffn_b200 import ops

    N, I, S, d = case
    idx, w, src, dy = make_case(dev, N, I, S, d, seed=3 * N + I)
    ref_dw = torch.zeros(N, I, device=dev)
    ref_gather.indexed_inner_product_fp32(idx, dy, src, ref_dw)
    dw = ops.indexed_inner_product(idx, dy, src)
    ref_dt = torch.zeros(S, d, device=dev)
    ref_gather.weighted_vector_scatter_add_fp32(idx, dy, w, ref_dt)
    dt = ops.weighted_vector_scatter_add(idx, dy, w, S)
    torch.cuda.synchronize()
    assert rel_err(dw.cpu(), ref_dw.cpu()) < 1e-5
    assert rel_err(dt.cpu(), ref_dt.cpu()) < 1e-4


@pytest.mark.parametrize("D", [64, 256, 512, 1024])
def test_fwht_fp32_bit_exact_against_reference_kernel(dev, ref_fht, D):
    from lookupffn_b200 import ops

    g = torch.Generator(device=dev).manual_seed(D)
    x = torch.randn(300, D, generator=g, device=dev)
    ref = ref_fht.fast_hadamard_transform(x)
    out = ops.fast_hadamard_transform(x)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


@pytest.mark.parametrize("D", [512, 1024])
def test_fwht_against_reference_fp16_kernels(dev, ref_fht, D):
    from lookupffn_b200 import ops

    g = torch.Generator(device=dev).manual_seed(D + 1)
    x16 = (torch.randn(256, D, generator=g, device=dev) / 8).half().contiguous()
    fn = ref_fht.fast_hadamard_transform_dim512_fp16 if D == 512 else ref_fht.fast_hadamard_transform_dim1024_fp16
    ref = fn(x16)
    out = ops.fast_hadamard_transform(x16.float())
    torch.cuda.synchronize()
    assert rel_err(ref.float().cpu(), out.cpu()) < 2e-2


def test_layer_against_reference_style_gpu_path(dev, ref_fht, ref_gather):
    """The whole layer against the reference's GPU evaluation (torch.einsum + its Hadamard and gather kernels +
    elementwise torch, oracle/ref_gpu_path.py).  einsum sums in another order than the fused kernel's fmaf chain, so
    z agrees to rounding, codes may differ only on coordinates with |v| < 1e-6, and tokens without such a
    coordinate get the same output to 1e-3 (the fp32 bound of the task)."""
    from argparse import Namespace

    from lookupffn_b200 import ops
    from lookupffn_b200.lookup import LookupFFN
    from oracle import ref_gpu_path as RG

    torch.manual_seed(3)
    cfg = Namespace(hidden_size=512, ffn_num_table=64, ffn_table_size=256, layer_norm_eps=1e-5, projection_type="bh4",
                    block_size=64)
    mod = LookupFFN(cfg, 512).to(dev).eval()
    with torch.no_grad():
        mod.hash.projection.bias.normal_(0, 0.05)
    x = torch.randn(4, 50, 512, device=dev)
    with torch.inference_mode():
        h = mod.LayerNorm(x.reshape(-1, 512))
        z_ref = RG.projection_reference_gpu(h, mod.hash.projection.weight, mod.hash.projection.bias, 64 * 8, ref_fht)
        z = mod.hash.projection(h)
        assert rel_err(z.cpu(), z_ref.cpu()) < 2e-5
        code_ref, score_ref = RG.code_score_reference_gpu(z.reshape(-1, 64, 8))
        code, score = ops.compute_code_score(z.reshape(-1, 64, 8).contiguous())
        assert torch.equal(code, code_ref)                       # same z in: identical codes
        assert rel_err(score.cpu(), score_ref.cpu()) < 1e-5
        # signs against the reference's GPU evaluation: only coordinates with |v| < 1e-6 (fp64 v) may differ
        from oracle import parity as PAR

        z64 = PAR.projection_fp64_torch(h, mod.hash.projection.weight, mod.hash.projection.bias, 64 * 8)
        rep, _ = PAR.assert_codes_match_up_to_tiny_coordinates(z.cpu().numpy(), z_ref.cpu().numpy(), z64.cpu().numpy())
        flipped = ((z > 0) != (z_ref > 0))
        y = mod(x).reshape(-1, 512)
        y_ref = RG.lookupffn_reference_gpu(mod, x, ref_fht, ref_gather).reshape(-1, 512)
        clean = ~flipped.any(dim=-1)
        assert int(clean.sum()) >= 190
        assert rel_err(y[clean].cpu(), y_ref[clean].cpu()) < 1e-3
