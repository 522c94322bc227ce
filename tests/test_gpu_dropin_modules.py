"""GPU test of the drop-in boundary the way the reference's Python code uses it: `decdec_ext` wrapped
in torch.library custom ops (as end-to-end/plugin.py:7-71 does) and called from Linear modules that follow
end-to-end/LUTGEMMLinear.py:85-102 and end-to-end/APLinear.py:36-58 (decode: clear the output buffer, fused
call; prefill: dequantise + matmul).  The reference tree is not present on the test machine, so the thin
modules below are written from its interfaces; the checks are against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import forward as ofw
from tests import problems as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def plugin():
    assert torch.cuda.is_available()
    import decdec_ext

    class Plugin:
        pass

    p = Plugin()

    @torch.library.custom_op("decdec_b200_test::dec_lutgemm", mutates_args={"output"})
    def dec_lutgemm(dec_config: int, x: torch.Tensor, output: torch.Tensor, q_weight: torch.Tensor, alpha: torch.Tensor,
                    q_bias: torch.Tensor, bitwidth: int, group_size: int) -> None:
        decdec_ext.dec_lutgemm(dec_config, x, output, q_weight, alpha, q_bias, bitwidth, group_size)

    @dec_lutgemm.register_fake
    def _(dec_config, x, output, q_weight, alpha, q_bias, bitwidth, group_size):
        return None

    @torch.library.custom_op("decdec_b200_test::dec_anyprec", mutates_args={"output"})
    def dec_anyprec(dec_config: int, x: torch.Tensor, output: torch.Tensor, q_weight: torch.Tensor, lut: torch.Tensor,
                    bitwidth: int) -> None:
        decdec_ext.dec_anyprec(dec_config, x, output, q_weight, lut, bitwidth)

    @dec_anyprec.register_fake
    def _(dec_config, x, output, q_weight, lut, bitwidth):
        return None

    p.ext, p.dec_lutgemm, p.dec_anyprec = decdec_ext, dec_lutgemm, dec_anyprec
    return p


class _Linear(torch.nn.Module):
    """Common part of the reference's DECLinear (end-to-end/DECLinear.py:20-43)."""

    def load_dec_data(self, q_residual, scales, thresholds):
        assert q_residual.dtype == torch.int and q_residual.shape == (self.in_features, self.out_features // 8)
        assert scales.shape == (self.out_features,) and thresholds.shape == (self.in_features,)
        self.q_residual, self.scales, self.thresholds = q_residual, scales, thresholds

    def create_dec_config(self, ext, ctx, k_chunk):
        self.dec_config = ext.create_dec_config(ctx, k_chunk, self.q_residual, self.scales, self.thresholds)


class LutLinear(_Linear):
    def __init__(self, plugin, L, K, N, bits, group):
        super().__init__()
        self.p, self.in_features, self.out_features, self.bitwidth, self.group_size = plugin, K, N, bits, group
        self.register_buffer("qweight", L["qweight"].cuda())
        self.register_buffer("alpha", L["alpha"].cuda())
        self.register_buffer("q_bias", L["q_bias"].cuda())
        self.output = torch.zeros((1, 1, N), dtype=torch.half, device="cuda")

    def forward(self, x):
        self.output.zero_()
        self.p.dec_lutgemm(self.dec_config, x, self.output, self.qweight, self.alpha, self.q_bias, self.bitwidth, self.group_size)
        return self.output


class ApLinear(_Linear):
    def __init__(self, plugin, L, K, N, bits):
        super().__init__()
        self.p, self.in_features, self.out_features, self.bitwidth = plugin, K, N, bits
        self.register_buffer("qweight", L["qweight"].cuda())
        self.register_buffer("lut", L["lut"].cuda())
        self.output = torch.zeros((1, 1, N), dtype=torch.half, device="cuda")

    def forward(self, x):
        if x.shape[1] > 1:                                   # prefill: dequantise + GEMM
            w = self.p.ext.anyprec_dequant(self.qweight, self.lut, self.bitwidth)
            return torch.matmul(x, w.T)
        self.output.zero_()
        self.p.dec_anyprec(self.dec_config, x, self.output, self.qweight, self.lut, self.bitwidth)
        return self.output


def test_reference_style_modules_decode_and_prefill(plugin):
    K, N, k_chunk = 2048, 512, 16
    ext = plugin.ext
    rows = torch.empty(32 * 1024, dtype=torch.int, device="cuda")          # model.py:168-173: one shared context
    acts = torch.empty(32 * 1024, dtype=torch.half, device="cuda")
    ctx = ext.create_dec_context(16, rows, acts)
    Lb = P.bcq_layer(N, K, 3, 128, seed=3)
    La = P.lut_layer(N, K, 3, seed=4)
    thr = P.make_thresholds(K)
    mods = []
    for kind, L in (("lut", Lb), ("ap", La)):
        cs, rs = P.random_residual(N, K, seed=5 if kind == "lut" else 6)
        m = LutLinear(plugin, L, K, N, 3, 128) if kind == "lut" else ApLinear(plugin, L, K, N, 3)
        m.load_dec_data(cs, rs, thr)
        m.create_dec_config(ext, ctx, k_chunk)
        mods.append((m, L, cs, rs))
    xbuf = torch.zeros(1, 1, K, dtype=torch.half, device="cuda")
    for m, *_ in mods:
        m(xbuf)                                                # eager warm-up (allocates the library workspace)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):                                  # generate.py:115-120 captures the decode step
        outs = [m(xbuf) for m, *_ in mods]
    for seed in (11, 12):
        x = P.make_activation(K, seed=seed)
        xbuf.copy_(x.cuda())
        g.replay()
        torch.cuda.synchronize()
        exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, "fp16")
        for (m, L, cs, rs), y in zip(mods, outs):
            delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
            ma, rl = P.errors(y, ofw.layer_output(L["w_hat"], P.to_np(x), None, delta))
            assert ma <= 1e-2 and rl <= 1e-3, (type(m).__name__, ma, rl)
    # prefill path of the any-precision module: [1, S, K] @ dequant(W)^T
    xs = torch.randn(1, 5, K, generator=torch.Generator().manual_seed(1)).half()
    y = mods[1][0](xs.cuda())
    ref = P.to_np(xs)[0] @ La["w_hat"].T
    assert np.abs(P.to_np(y)[0] - ref).max() <= 3e-2
    # re-tune: new context object, new k_chunk, no re-upload (profiler.py:74-84 -> model.py:175-198)
    ctx2 = ext.create_dec_context(8, rows, acts)
    for m, *_ in mods:
        ext.update_dec_config(m.dec_config, ctx2, 8)
    x = P.make_activation(K, seed=13)
    y = mods[0][0](x.cuda())
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, 8, "fp16")
    delta = ofw.dec_delta(P.to_np(x), exp_rows, mods[0][2].numpy(), P.to_np(mods[0][3]), exp_acts)
    ma, rl = P.errors(y, ofw.layer_output(Lb["w_hat"], P.to_np(x), None, delta))
    assert ma <= 1e-2 and rl <= 1e-3


def test_artifact_file_formats_roundtrip(tmp_path):
    """cheatsheet.pt / thresholds.pt as written by decdec_setup (cheatsheet.py:239, thresholds.py:208): lists over
    layers of dicts keyed by module name; the tensors load back into create_dec_config unchanged."""
    import decdec_ext as ext
    K, N = 1024, 64
    cs, rs = P.random_residual(N, K, seed=1)
    thr32 = P.make_thresholds(K).float()
    torch.save([{"self_attn.o_proj": {"cheatsheet": cs, "reordered_scales": rs}}], tmp_path / "cheatsheet.pt")
    torch.save([{"self_attn.o_proj": thr32}], tmp_path / "thresholds.pt")
    c = torch.load(tmp_path / "cheatsheet.pt")[0]["self_attn.o_proj"]
    t = torch.load(tmp_path / "thresholds.pt")[0]["self_attn.o_proj"].half()
    rows = torch.zeros(256, dtype=torch.int32, device="cuda")
    acts = torch.zeros(256, dtype=torch.half, device="cuda")
    ctx = ext.create_dec_context(4, rows, acts)
    cfg = ext.create_dec_config(ctx, 8, c["cheatsheet"], c["reordered_scales"], t)
    x = P.make_activation(K, seed=2)
    y = torch.zeros(1, 1, N, dtype=torch.half, device="cuda")
    ext.dec(cfg, x.cuda(), y)
    torch.cuda.synchronize()
    exp_rows, exp_acts, _ = P.expected_selection(x, t, 8, "fp16")
    assert np.array_equal(rows[:8].cpu().numpy(), exp_rows)
    ma, rl = P.errors(y, ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts))
    assert rl <= 1e-3
    ext.destroy_dec_config(cfg)
