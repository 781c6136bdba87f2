"""Generate tests/golden/lookupffn_golden.npz by running the REFERENCE's own code.

Run in a container that has the reference checkout (its location is taken from LFFN_REFERENCE_ROOT when set)
after `python oracle/build.py`:

    python tests/golden/make_golden.py

The reference ships no golden vectors, so these are produced by importing its
Python modules and calling them on seeded inputs.  What is executed, per group:

  ccs_*      compute_code_score_torch (compute_code_score/kernel.py:43-55) and the C++
             extension ccs_cpu.compute_code_score (torch_extension.cc:14-42), the latter from
             the unmodified source compiled into oracle/_ref by oracle/build.py
  had_*      hadamard_transform (bh4/fast_hadamard_transform/kernel.py:31-37)
  bh4_*      bh4_cuda (bh4/kernel.py:23-36) and BH4._forward (lookup.py:29-39) on CPU tensors,
             with `hadamard` bound to the reference's own hadamard_transform because its
             CUDA kernels cannot run without a GPU
  gat_*      weighted_vector_gather_add(use_torch=True) (gather/cpu/kernel.py:28-64) and the
             C++ weighted_vector_gather_add_scalar / _avx2_par (gather/cpu/torch_extension.cpp)
  bwd_*      indexed_inner_product(use_torch=True), weighted_vector_scatter_add(use_torch=True)
             and WeightedVectorGatherAdd's torch path (gather/cuda/kernel.py:72-173)
  enc_*      Lookup.forward (encoder.py:21-32), eval, 2 layers, on CPU, same bindings as mod_*
  mod_*      LookupFFN.forward (lookup.py:79-129), eval, on CPU, for projection_type "dense"
             and "bh4"; bh4/gather dispatch bound to the functions above because the
             reference's CPU wrappers assert one fixed shape and need libxsmm

torch.utils.cpp_extension.load is replaced by a loader that returns the prebuilt
oracle/_ref modules (and inert stand-ins for the two CUDA extensions, which are
never called here), so nothing is JIT-compiled.
"""
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
# the reference checkout: LFFN_REFERENCE_ROOT, else a directory named "reference" beside this repository
REF = os.environ.get("LFFN_REFERENCE_ROOT") or os.path.join(os.path.dirname(REPO), "reference")
OUT = os.path.join(HERE, "lookupffn_golden.npz")

sys.path.insert(0, REPO)
sys.path.insert(0, REF)
sys.dont_write_bytecode = True

import torch  # noqa: E402
import torch.utils.cpp_extension as cpp_ext  # noqa: E402

from oracle import build as obuild  # noqa: E402


def _install_loader():
    import importlib.util

    def load(name, sources=None, *a, **k):
        path = obuild.ref_module_path(name)
        if os.path.exists(path):
            spec = importlib.util.spec_from_file_location(name, path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
        else:
            mod = types.ModuleType(name)  # CUDA extensions: imported, never called on CPU
        sys.modules[name] = mod
        return mod

    cpp_ext.load = load


def main():
    torch.manual_seed(0)
    torch.set_num_threads(4)
    obuild.build_ref(verbose=False)
    _install_loader()

    from argparse import Namespace

    import src.roberta.models.prenorm_lookup.lookup as ref_lookup
    import src.roberta.models.prenorm_lookup.bh4.kernel as ref_bh4
    import src.roberta.models.prenorm_lookup.bh4.fast_hadamard_transform.kernel as ref_fht
    import src.roberta.models.prenorm_lookup.compute_code_score.kernel as ref_ccs
    import src.roberta.models.prenorm_lookup.gather.cpu.kernel as ref_gcpu
    import src.roberta.models.prenorm_lookup.gather.cuda.kernel as ref_gcuda

    # the CUDA Hadamard kernels cannot run here: use the reference's own matmul definition
    ref_bh4.hadamard = lambda y: ref_fht.hadamard_transform(y.contiguous())

    rng = np.random.RandomState(20240607)
    g = {}

    # ---- code + score -------------------------------------------------------------------
    for tag, (N, T, k) in {"k8": (96, 12, 8), "k6": (40, 10, 6), "k10": (24, 5, 10), "k1": (8, 4, 1)}.items():
        z = rng.randn(N, T, k).astype(np.float32)
        z[0, 0, :] = 0.0
        z[1, 0, 0] = -0.0
        z[2, 1, :3] = np.array([1e-30, -1e-30, 1e-7], dtype=np.float32)[:min(3, k)]
        z[3, 2, 0] = 30.0
        zt = torch.from_numpy(z)
        c_t, s_t = ref_ccs.compute_code_score_torch(zt)
        c_c, s_c = ref_ccs.compute_code_score_cpu(zt)
        g[f"ccs_{tag}_z"] = z
        g[f"ccs_{tag}_code_torch"] = c_t.numpy()
        g[f"ccs_{tag}_score_torch"] = s_t.numpy()
        g[f"ccs_{tag}_code_cpp"] = c_c.numpy()
        g[f"ccs_{tag}_score_cpp"] = s_c.numpy()

    # ---- Hadamard --------------------------------------------------------------------------
    for D in (64, 256, 1024):
        x = rng.randn(6, D).astype(np.float32)
        g[f"had_{D}_x"] = x
        g[f"had_{D}_y"] = ref_fht.hadamard_transform(torch.from_numpy(x)).numpy()

    # ---- bh4_cuda and BH4 module ---------------------------------------------------------
    for tag, (N, in_dim, out_dim, BS) in {"a": (20, 128, 256, 64), "b": (12, 100, 200, 64),
                                           "c": (10, 256, 160, 64), "d": (9, 60, 150, 16)}.items():
        mod = ref_lookup.BH4(in_dim, out_dim, BS)
        with torch.no_grad():
            mod.bias.copy_(torch.from_numpy((0.05 * rng.randn(out_dim)).astype(np.float32)))
            mod.weight.copy_(torch.from_numpy(
                (rng.randn(*mod.weight.shape) / np.sqrt(BS * mod.padded_in_dim)).astype(np.float32)))
        mod.train()  # training=True routes to bh4_cuda; the is_cuda asserts are bypassed below
        x = rng.randn(N, in_dim).astype(np.float32)
        xt = torch.from_numpy(x)
        D = mod.padded_in_dim
        xp = torch.cat([xt, torch.zeros(N, D - in_dim)], dim=-1) if in_dim < D else xt
        with torch.no_grad():
            P = ref_bh4.bh4_cuda(xp.contiguous(), mod.weight)
            ref_lookup.bh4 = lambda x_, w_, training: ref_bh4.bh4_cuda(x_, w_)
            z = mod(xt)
        g[f"bh4_{tag}_x"] = x
        g[f"bh4_{tag}_w"] = mod.weight.detach().numpy().copy()
        g[f"bh4_{tag}_bias"] = mod.bias.detach().numpy().copy()
        g[f"bh4_{tag}_P"] = P.numpy()
        g[f"bh4_{tag}_z"] = z.numpy()
        g[f"bh4_{tag}_meta"] = np.array([in_dim, out_dim, BS, D, mod.num_repeat], dtype=np.int64)

    # ---- gather forward ---------------------------------------------------------------------
    # shape valid for the reference's tiled C++ kernel: one index per table, 256-row tables, N % 64 == 0
    N, T, rows, d = 64, 6, 256, 64
    idx = (rng.randint(0, rows, size=(N, T)) + np.arange(T)[None] * rows).astype(np.int32)
    w = rng.randn(N, T).astype(np.float32)
    tab = (0.02 * rng.randn(T * rows, d)).astype(np.float32)
    it, wt, tt = torch.from_numpy(idx), torch.from_numpy(w), torch.from_numpy(tab)
    import gather_add_cpu
    g["gat_a_idx"], g["gat_a_w"], g["gat_a_tables"] = idx, w, tab
    g["gat_a_out_torch"] = ref_gcpu.weighted_vector_gather_add(it, tt, wt, use_torch=True).numpy()
    g["gat_a_out_scalar"] = gather_add_cpu.weighted_vector_gather_add_scalar(it, tt, wt).numpy()
    g["gat_a_out_avx2"] = gather_add_cpu.weighted_vector_gather_add_avx2_par(it, tt, wt).numpy()
    # generic index list (repeats, any row), only the scalar kernel and the torch path are valid
    N, I, S, d = 40, 18, 333, 128
    idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
    idx[0, :] = 7
    w = rng.randn(N, I).astype(np.float32)
    tab = (0.02 * rng.randn(S, d)).astype(np.float32)
    it, wt, tt = torch.from_numpy(idx), torch.from_numpy(w), torch.from_numpy(tab)
    g["gat_b_idx"], g["gat_b_w"], g["gat_b_tables"] = idx, w, tab
    g["gat_b_out_torch"] = ref_gcpu.weighted_vector_gather_add(it, tt, wt, use_torch=True).numpy()
    g["gat_b_out_scalar"] = gather_add_cpu.weighted_vector_gather_add_scalar(it, tt, wt).numpy()

    # ---- gather backward ----------------------------------------------------------------------
    N, I, S, d = 32, 8, 300, 64
    idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
    idx[:4, :] = 5
    w = rng.randn(N, I).astype(np.float32)
    tab = (0.02 * rng.randn(S, d)).astype(np.float32)
    dy = rng.randn(N, d).astype(np.float32)
    it, wt, tt, dyt = map(torch.from_numpy, (idx, w, tab, dy))
    g["bwd_idx"], g["bwd_w"], g["bwd_tables"], g["bwd_dy"] = idx, w, tab, dy
    g["bwd_dw"] = ref_gcuda.indexed_inner_product(it, dyt, tt, use_torch=True).numpy()
    g["bwd_dtables"] = ref_gcuda.weighted_vector_scatter_add(it, dyt, wt, S, use_torch=True).numpy()
    # the same two gradients through autograd of the reference's torch forward
    tt2 = tt.clone().requires_grad_(True)
    wt2 = wt.clone().requires_grad_(True)
    out = ref_gcuda.weighted_gather_add(it, tt2, wt2, use_torch=True)
    out.backward(dyt)
    g["bwd_out"] = out.detach().numpy()
    g["bwd_dw_autograd"] = wt2.grad.numpy()
    g["bwd_dtables_autograd"] = tt2.grad.numpy()

    # ---- whole module --------------------------------------------------------------------------
    ref_lookup.gather = lambda indices, weights, tables, training: ref_gcpu.weighted_vector_gather_add(
        indices, tables, weights, use_torch=True)
    for tag, cfg in {
        "dense": dict(hidden_size=96, ffn_num_table=10, ffn_table_size=64, projection_type="dense", block_size=64),
        "bh4": dict(hidden_size=96, ffn_num_table=24, ffn_table_size=256, projection_type="bh4", block_size=64),
    }.items():
        config = Namespace(layer_norm_eps=1e-5, **cfg)
        out_size = 32
        mod = ref_lookup.LookupFFN(config, out_size)
        with torch.no_grad():
            for name, p in mod.named_parameters():
                if name in ("LayerNorm.weight",):
                    p.copy_(torch.from_numpy((1 + 0.1 * rng.randn(*p.shape)).astype(np.float32)))
                elif name in ("LayerNorm.bias", "hash.projection.bias"):
                    p.copy_(torch.from_numpy((0.05 * rng.randn(*p.shape)).astype(np.float32)))
        mod.eval()
        x = rng.randn(3, 8, config.hidden_size).astype(np.float32)  # two leading dims (lookup.py:112-118)
        with torch.no_grad():
            xt = torch.from_numpy(x)
            y = mod(xt)
            u = mod.LayerNorm(xt.reshape(-1, config.hidden_size))
            z = mod.hash.projection(u)
            code, score = mod.hash(u)
        for name, p in mod.state_dict().items():
            g[f"mod_{tag}_param_{name}"] = p.numpy().copy()
        g[f"mod_{tag}_x"] = x
        g[f"mod_{tag}_u"] = u.numpy()
        g[f"mod_{tag}_z"] = z.numpy()
        g[f"mod_{tag}_code"] = code.numpy()
        g[f"mod_{tag}_score"] = score.numpy()
        g[f"mod_{tag}_y"] = y.numpy()

    # ---- the Lookup encoder (the caller of the layer): layer.py:66-78, encoder.py:9-37 -----------------
    import src.roberta.models.prenorm_lookup.encoder as ref_encoder

    cfg = Namespace(vocab_size=120, type_vocab_size=1, pad_token_id=1, num_hidden_layers=2, num_attention_heads=4,
                    attention_head_size=16, layer_norm_eps=1e-5, hidden_size=64, hidden_dropout_prob=0.1,
                    attention_probs_dropout_prob=0.1, max_position_embeddings=32, projection_type="bh4",
                    block_size=64, ffn_num_table=12, ffn_table_size=16, intermediate_size=256,
                    initializer_range=0.02)
    enc = ref_encoder.Lookup(cfg)
    enc.eval()
    B, S = 3, 24  # B*S a multiple of 8: the reference torch gather works in mini-batches of 8
    ids = rng.randint(5, cfg.vocab_size, size=(B, S)).astype(np.int64)
    ids[:, 0] = 0
    mask = np.ones((B, S), dtype=np.float32)
    mask[1, 17:] = 0.0
    with torch.no_grad():
        out, _ = enc(torch.from_numpy(ids), torch.zeros(B, S, dtype=torch.long),
                     torch.arange(S)[None].repeat(B, 1), torch.from_numpy(mask))
    for name, p in enc.state_dict().items():
        g[f"enc_param_{name}"] = p.numpy().copy()
    g["enc_ids"], g["enc_mask"], g["enc_out"] = ids, mask, out.numpy()

    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
