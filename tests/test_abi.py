"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the header
declares, and rejects bad arguments with an error code and message before touching a GPU."""
import ctypes as C
import os
import re

import pytest
import torch

from lookupffn_b200 import _lib as L

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(REPO, "include", "lookupffn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lffn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = L.lib()
    names = declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/lookupffn.h but not exported"
    # and the Python binding covers each of them
    assert set(names) == set(L.exported_symbols())


def test_version_and_error_string():
    lib = L.lib()
    assert lib.lffn_version() == 100
    assert isinstance(lib.lffn_last_error_string(), bytes)


def test_hash_desc_layout_matches_header():
    # 14 four-byte fields then two pointers: 72 bytes on LP64
    assert C.sizeof(L.HashDesc) == 14 * 4 + 2 * 8
    assert L.HashDesc.proj_w.offset == 56


def test_argument_errors_are_reported_not_raised_by_cuda():
    lib = L.lib()
    rc = lib.lffn_gather_fwd(None, None, None, 0, None, 0, 4, 2, 8, 64, None, None)
    assert rc == -1 and b"NULL" in lib.lffn_last_error_string()
    assert lib.lffn_gather_fwd(None, None, None, 0, None, 0, 0, 2, 8, 64, None, None) == 0  # no tokens: nothing to do
    buf = (C.c_float * 64)()
    p = C.cast(buf, C.c_void_p)
    rc = lib.lffn_gather_fwd(p, p, p, 0, p, 0, 4, 2, 8, 6, None, None)  # d not a multiple of 4
    assert rc == -2 and b"multiple" in lib.lffn_last_error_string()
    rc = lib.lffn_gather_fwd(p, p, p, 7, p, 0, 4, 2, 8, 64, None, None)  # bad dtype
    assert rc == -1
    desc = L.HashDesc(d_in=100, D=128, BS=1, S=2, R=1, T=40, k=8, proj_w=1)  # R*D < T*k
    rc = lib.lffn_hash_fwd(C.byref(desc), p, 0, 4, 0, 40, p, p, None, None)
    assert rc == -1 and b"R*D" in lib.lffn_last_error_string()
    desc = L.HashDesc(d_in=100, D=128, BS=1, S=2, R=3, T=40, k=8, proj_w=1)
    rc = lib.lffn_hash_fwd(C.byref(desc), p, 0, 4, 30, 20, p, p, None, None)  # table range outside T
    assert rc == -1 and b"table range" in lib.lffn_last_error_string()
    desc = L.HashDesc(d_in=100, D=128, BS=1, S=2, R=3, T=40, k=17, proj_w=1)
    assert lib.lffn_hash_fwd(C.byref(desc), p, 0, 4, 0, 40, p, p, None, None) == -2
    assert lib.lffn_gather_bwd_tables_sorted_scratch_bytes(16, 4, 1, 256) > 0
    with pytest.raises(L.LookupFFNError):
        L.check(-2)


def test_ops_refuse_cpu_tensors():
    from lookupffn_b200 import LookupFFN, ops
    from argparse import Namespace

    with pytest.raises(RuntimeError, match="CUDA"):
        ops.hadamard(torch.zeros(2, 64))
    cfg = Namespace(hidden_size=64, ffn_num_table=8, ffn_table_size=16, layer_norm_eps=1e-5,
                    projection_type="bh4", block_size=16)
    mod = LookupFFN(cfg, 32)
    assert set(mod.state_dict()) == {"LayerNorm.weight", "LayerNorm.bias", "hash.projection.weight",
                                     "hash.projection.bias", "tables", "bias"}
    assert mod.state_dict()["hash.projection.weight"].shape == (1, 4, 4, 16, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        mod(torch.zeros(3, 64))


def test_module_loads_reference_state_dict(golden):
    from argparse import Namespace
    from lookupffn_b200 import LookupFFN

    for tag, ptype in (("bh4", "bh4"), ("dense", "dense")):
        sd = {k[len(f"mod_{tag}_param_"):]: torch.from_numpy(v) for k, v in golden.items()
              if k.startswith(f"mod_{tag}_param_")}
        T, rows, d_out = sd["tables"].shape
        cfg = Namespace(hidden_size=sd["LayerNorm.weight"].numel(), ffn_num_table=T, ffn_table_size=rows,
                        layer_norm_eps=1e-5, projection_type=ptype, block_size=64)
        mod = LookupFFN(cfg, d_out)
        mod.load_state_dict(sd, strict=True)


def _encoder_config():
    from argparse import Namespace

    return Namespace(vocab_size=120, type_vocab_size=1, pad_token_id=1, num_hidden_layers=2, num_attention_heads=4,
                     attention_head_size=16, layer_norm_eps=1e-5, hidden_size=64, hidden_dropout_prob=0.1,
                     attention_probs_dropout_prob=0.1, max_position_embeddings=32, projection_type="bh4",
                     block_size=64, ffn_num_table=12, ffn_table_size=16)


def test_encoder_loads_reference_state_dict(golden):
    from lookupffn_b200.encoder import Lookup

    sd = {k[len("enc_param_"):]: torch.from_numpy(v) for k, v in golden.items() if k.startswith("enc_param_")}
    enc = Lookup(_encoder_config())
    assert set(enc.state_dict()) == set(sd)
    enc.load_state_dict(sd, strict=True)
