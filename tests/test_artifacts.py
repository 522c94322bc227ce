"""Artifact producers / loaders (decdec_b200/artifacts.py) against the reference's own output and the oracle.

tests/golden/cheatsheet.npz was produced by the reference's `decdec_setup/cheatsheet.py:_process_layer`
(generator: tests/golden/make_golden.py).  CPU only.
"""
import os

import numpy as np
import pytest
import torch

from decdec_b200 import artifacts as A
from oracle import residual as oracle_residual

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_layer_cheatsheet_matches_reference_bit_for_bit():
    d = np.load(os.path.join(G, "cheatsheet.npz"))
    w, wq = torch.from_numpy(d["w"]), torch.from_numpy(d["wq"])
    out = A.build_layer_cheatsheet({"proj": w}, {"proj": wq})["proj"]
    assert out["cheatsheet"].dtype == torch.int32 and tuple(out["cheatsheet"].shape) == (w.shape[1], w.shape[0] // 8)
    assert np.array_equal(out["cheatsheet"].numpy(), d["cheatsheet"])
    assert np.array_equal(out["reordered_scales"].numpy(), d["reordered_scales"])


def test_quantizer_and_packer_agree_with_oracle():
    g = torch.Generator().manual_seed(3)
    err = (torch.randn(24, 160, generator=g) * 0.003).half()
    codes, scales = A.quantize_residual(err)
    oq, osc = oracle_residual.quantize_residual(err)
    assert torch.equal(codes, oq) and torch.equal(scales, osc)
    q, rs = A.pack_cheatsheet(codes, scales)
    ocs, ors = oracle_residual.pack_cheatsheet(oq.numpy(), osc.numpy())
    assert np.array_equal(q.numpy(), ocs) and np.array_equal(rs.numpy(), ors)
    c2, s2 = A.unpack_cheatsheet(q, rs)
    assert torch.equal(c2.to(torch.int8), codes) and torch.equal(s2, scales)
    # extreme codes survive the signed 32-bit word
    codes2 = torch.randint(-8, 8, (16, 40), generator=g, dtype=torch.int8)
    q2, rs2 = A.pack_cheatsheet(codes2, scales[:16])
    assert torch.equal(A.unpack_cheatsheet(q2, rs2)[0].to(torch.int8), codes2)
    assert np.array_equal(q2.numpy(), oracle_residual.pack_cheatsheet(codes2.numpy(), scales[:16].numpy())[0])


def test_thresholds_statistic():
    g = torch.Generator().manual_seed(5)
    acts = torch.randn(37, 96, generator=g)
    acts[:, 7] *= 20
    t = A.thresholds_from_calibration(acts)
    assert np.allclose(t.numpy(), oracle_residual.thresholds_from_calibration(acts.numpy()))
    assert bool((t[:-1] >= t[1:]).all())                      # descending by construction
    acc = A.ThresholdAccumulator(96)
    acc.update(acts[:20].reshape(4, 5, 96))
    acc.update(acts[20:])
    assert torch.equal(acc.value, t)                           # batches in any split give the same statistic


def _part(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-7, 8, (n, k), generator=g, dtype=torch.int8)
    scales = (torch.rand(n, generator=g) * 1e-3 + 1e-4).half()
    q, rs = A.pack_cheatsheet(codes, scales)
    return {"cheatsheet": q, "reordered_scales": rs}


def test_fused_projections_keep_every_rows_scale():
    parts = [_part(32, 64, 1), _part(8, 64, 2), _part(16, 64, 3)]            # q, k, v of unequal width
    fused = A.fuse_projections(parts)
    dense = torch.cat([A.residual_matrix(p["cheatsheet"], p["reordered_scales"]) for p in parts], dim=0)
    assert torch.equal(A.residual_matrix(fused["cheatsheet"], fused["reordered_scales"]), dense)
    # concatenating the stored (nibble-major) scales, as end-to-end/loader.py:130-137 does, pairs rows with wrong scales
    naive = torch.cat([p["reordered_scales"] for p in parts], dim=0)
    assert not torch.equal(naive, fused["reordered_scales"])
    assert not torch.equal(A.residual_matrix(fused["cheatsheet"], naive), dense)
    # the sharding module's view of the layout agrees
    from decdec_b200 import tp
    assert torch.equal(tp.unreorder_scales(fused["reordered_scales"]), A.unreorder_scales(fused["reordered_scales"]))


def test_assemble_names_and_file_round_trip(tmp_path):
    K = 64
    layers = []
    thr_layers = []
    for i in range(2):
        layer = {"self_attn.q_proj": _part(32, K, 10 + i), "self_attn.k_proj": _part(8, K, 20 + i), "self_attn.v_proj": _part(8, K, 30 + i),
                 "self_attn.o_proj": _part(32, K, 40 + i), "mlp.gate_proj": _part(48, K, 50 + i), "mlp.up_proj": _part(48, K, 60 + i),
                 "mlp.down_proj": _part(K, 48 * 2, 70 + i)}
        layers.append(layer)
        thr_layers.append({m: torch.sort(torch.rand(layer[m]["cheatsheet"].shape[0]), descending=True).values for m in layer})
    A.save_cheatsheet(str(tmp_path / "cheatsheet.pt"), layers)
    A.save_thresholds(str(tmp_path / "thresholds.pt"), thr_layers)
    d = A.load(str(tmp_path / "cheatsheet.pt"), str(tmp_path / "thresholds.pt"))
    for i in range(2):
        for mod in ("attention.wqkv", "attention.wo", "feed_forward.w1w3", "feed_forward.w2"):      # w2 included
            for leaf in ("q_residual", "scales", "thresholds"):
                assert f"layers.{i}.{mod}.{leaf}" in d
        assert tuple(d[f"layers.{i}.attention.wqkv.q_residual"].shape) == (K, 48 // 8)
        assert tuple(d[f"layers.{i}.feed_forward.w1w3.q_residual"].shape) == (K, 96 // 8)
        assert torch.equal(d[f"layers.{i}.feed_forward.w2.q_residual"], layers[i]["mlp.down_proj"]["cheatsheet"])
        assert torch.equal(d[f"layers.{i}.attention.wqkv.thresholds"], thr_layers[i]["self_attn.q_proj"])
    # already fused input is passed through
    fused_layer = {"self_attn.qkv_proj": A.fuse_projections([layers[0][m] for m in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj")]),
                   "self_attn.o_proj": layers[0]["self_attn.o_proj"],
                   "mlp.gate_up_proj": A.fuse_projections([layers[0]["mlp.gate_proj"], layers[0]["mlp.up_proj"]]),
                   "mlp.down_proj": layers[0]["mlp.down_proj"]}
    d2 = A.assemble([fused_layer], [])
    assert torch.equal(d2["layers.0.attention.wqkv.scales"], d["layers.0.attention.wqkv.scales"])


def test_shape_errors():
    with pytest.raises(ValueError):
        A.pack_cheatsheet(torch.zeros(12, 8, dtype=torch.int8), torch.zeros(12))
    with pytest.raises(ValueError):
        A.quantize_residual(torch.zeros(8))
