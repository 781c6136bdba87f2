"""Checkpoint helpers: prefix stripping of a reference Lightning checkpoint, table conversion, row re-ordering
between code bit orders (checked with the CPU oracle: LSB codes on re-ordered tables = MSB codes on the originals)."""
import numpy as np
import pytest
import torch

from lookupffn_b200 import checkpoint as ck
from oracle import oracle as O


def test_strip_prefixes_and_load(golden, tmp_path):
    from tests.test_abi import _encoder_config
    from lookupffn_b200.encoder import Lookup

    enc_sd = {k[len("enc_param_"):]: torch.from_numpy(v) for k, v in golden.items() if k.startswith("enc_param_")}
    lightning = {"state_dict": {**{"model.roberta." + k: v for k, v in enc_sd.items()},
                                "model.lm_head.dense.weight": torch.zeros(2, 2)}, "epoch": 3}
    path = tmp_path / "last.ckpt"
    torch.save(lightning, path)
    sd = ck.encoder_state_dict(str(path))
    assert set(sd) == set(enc_sd)
    Lookup(_encoder_config()).load_state_dict(sd, strict=True)
    layer = ck.layer_state_dict(sd, 1)
    assert set(layer) == {"LayerNorm.weight", "LayerNorm.bias", "hash.projection.weight", "hash.projection.bias",
                          "tables", "bias"}
    with pytest.raises(KeyError):
        ck.encoder_state_dict({"state_dict": {"foo": torch.zeros(1)}})
    half = ck.tables_to(sd)
    assert half["encoder.layer.0.FFN.tables"].dtype == torch.bfloat16
    assert half["encoder.layer.0.FFN.bias"].dtype == torch.float32


def test_bit_order_reordering_is_consistent_with_the_oracle():
    rng = np.random.RandomState(1)
    T, k, d, N = 5, 6, 8, 40
    z = rng.randn(N, T * k).astype(np.float32)
    tables = rng.randn(T, 1 << k, d).astype(np.float32)
    idx_m, w = O.code_weights(z, T, k, bit_order=O.MSB_FIRST)
    idx_l, _ = O.code_weights(z, T, k, bit_order=O.LSB_FIRST)
    re = ck.reorder_tables_bit_order(torch.from_numpy(tables))
    y_m = O.gather(idx_m, w, tables.reshape(-1, d))
    y_l = O.gather(idx_l, w, re.numpy().reshape(-1, d))
    np.testing.assert_array_equal(y_m, y_l)
    assert torch.equal(ck.reorder_tables_bit_order(re), torch.from_numpy(tables))
    assert ck.bit_reverse_permutation(3).tolist() == [0, 4, 2, 6, 1, 5, 3, 7]
