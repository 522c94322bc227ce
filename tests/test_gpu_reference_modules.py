"""The reference's own Python consumers of the binding, run UNCHANGED on top of this repository's `decdec_ext`.

`oracle/build_ref.py` places end-to-end/{plugin,DECLinear,APLinear,LUTGEMMLinear}.py of a reference checkout
under oracle/_ref/ref_modules/ (not tracked).  They are imported as they are: `plugin.py` wraps `decdec_ext`
in torch.library custom ops with fakes (plugin.py:7-71), the Linear classes clear their output buffer and
make one fused call per decode step (LUTGEMMLinear.py:85-102, APLinear.py:36-58) and dequantize + matmul for
prefill.  A two-layer decode step is run eagerly, captured in a CUDA graph (generate.py:115-120) and under
torch.compile(fullgraph=True) (generate.py:311), and checked against the CPU oracle.
"""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import forward as ofw
from tests import problems as P

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODS = os.path.join(ROOT, "oracle", "_ref", "ref_modules")

K0, N0, N1, KC = 2048, 1024, 256, 16


@pytest.fixture(scope="module")
def ref_mods():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    if not os.path.exists(os.path.join(MODS, "plugin.py")):
        pytest.skip("reference modules absent: run `python oracle/build_ref.py <DecDEC checkout>` first")
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)            # `import decdec_ext` inside plugin.py finds this repository's module
    sys.path.insert(0, MODS)
    try:
        import plugin
        import APLinear
        import LUTGEMMLinear
    finally:
        sys.path.remove(MODS)
    import decdec_ext
    assert os.path.dirname(os.path.abspath(decdec_ext.__file__)) == ROOT
    return plugin, LUTGEMMLinear.LUTGEMMLinear, APLinear.APLinear


@pytest.fixture(scope="module")
def model(ref_mods):
    plugin, LUTGEMMLinear, APLinear = ref_mods
    rows = torch.zeros(32 * 1024, dtype=torch.int32, device="cuda")
    acts = torch.zeros(32 * 1024, dtype=torch.float16, device="cuda")
    ctx = plugin.create_dec_context(12, rows, acts)

    Lb = P.bcq_layer(N0, K0, 3, 128, seed=101)
    l0 = LUTGEMMLinear(K0, N0, 3, 128)
    l0.qweight.copy_(Lb["qweight"]); l0.alpha.copy_(Lb["alpha"]); l0.q_bias.copy_(Lb["q_bias"])
    cs0, rs0 = P.quantized_residual(Lb["w"], Lb["w_fake"])
    thr0 = P.make_thresholds(K0)
    l0.load_dec_data(cs0, rs0, thr0)
    l0.create_dec_config(ctx, KC)

    La = P.lut_layer(N1, N0, 3, seed=102)
    l1 = APLinear(N0, N1, 3)
    l1.qweight.copy_(La["qweight"]); l1.lut.copy_(La["lut"])
    cs1, rs1 = P.random_residual(N1, N0, seed=103)
    thr1 = torch.sort(torch.rand(N0, generator=torch.Generator().manual_seed(5)) * 4, descending=True).values.half()
    l1.load_dec_data(cs1, rs1, thr1)
    l1.create_dec_config(ctx, KC)

    def step(x):
        h = l0(x)
        return l1(torch.nn.functional.silu(h))

    def expected(x):
        """Float64 value of the two layers, the second fed with the fp16 activations the first produced."""
        r0, a0, _ = P.expected_selection(x, thr0, KC, "fp16")
        y0 = ofw.layer_output(Lb["w_hat"], P.to_np(x), None, ofw.dec_delta(P.to_np(x), r0, cs0.numpy(), P.to_np(rs0), a0))
        h = torch.nn.functional.silu(torch.from_numpy(y0).half().reshape(1, 1, N0))
        return y0, h

    def expected_second(h):
        r1, a1, _ = P.expected_selection(h, thr1, KC, "fp16")
        return ofw.layer_output(La["w_hat"], P.to_np(h), None, ofw.dec_delta(P.to_np(h), r1, cs1.numpy(), P.to_np(rs1), a1))

    return dict(step=step, l0=l0, l1=l1, expected=expected, expected_second=expected_second, ctx=ctx, plugin=plugin,
                keep=(rows, acts), Lb=Lb, La=La)


def _check(model, x, out, what):
    y0_ref, _ = model["expected"](x)
    ma, rl = P.errors(model["l0"].output, y0_ref)
    assert ma <= 1e-2 and rl <= 1e-3, f"{what}: first layer max abs {ma:.2e} rel {rl:.2e}"
    # second layer against the oracle fed with the activations the GPU actually produced
    h_gpu = torch.nn.functional.silu(model["l0"].output).cpu()
    y1_ref = model["expected_second"](h_gpu)
    ma, rl = P.errors(out, y1_ref)
    assert ma <= 1e-2 and rl <= 2e-3, f"{what}: second layer max abs {ma:.2e} rel {rl:.2e}"


def test_reference_modules_decode_eager(model):
    for seed in (1, 2):
        x = P.make_activation(K0, seed=seed)
        out = model["step"](x.cuda())
        torch.cuda.synchronize()
        _check(model, x, out, f"eager seed {seed}")


def test_reference_modules_prefill(model):
    """Sequence length > 1 takes the dequantize + matmul branch of the reference modules
    (LUTGEMMLinear.py:41-82 in torch ops; APLinear.py:36-39 through decdec_ext.anyprec_dequant)."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1, 5, K0, generator=g).half().cuda()
    y = model["l0"](x)
    ref = P.to_np(x).reshape(5, K0) @ model["Lb"]["w_hat"].T
    assert np.abs(P.to_np(y).reshape(5, N0) - ref).max() <= 5e-2
    x1 = torch.randn(1, 5, N0, generator=g).half().cuda()
    y1 = model["l1"](x1)
    ref1 = P.to_np(x1).reshape(5, N0) @ model["La"]["w_hat"].T
    assert np.abs(P.to_np(y1).reshape(5, N1) - ref1).max() <= 5e-2


def test_reference_modules_cuda_graph(model):
    xbuf = P.make_activation(K0, seed=4).cuda()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        model["step"](xbuf)              # first call on the capture stream happens outside capture
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = model["step"](xbuf)
    for seed in (5, 6, 7):
        x = P.make_activation(K0, seed=seed)
        xbuf.copy_(x.cuda())
        g.replay()
        torch.cuda.synchronize()
        _check(model, x, out, f"graph replay seed {seed}")


@pytest.mark.parametrize("backend", ["aot_eager", "inductor"])
def test_reference_modules_torch_compile_fullgraph(model, backend):
    """The reference compiles its decode step with fullgraph=True (generate.py:311); the custom ops must trace through
    their fakes and the compiled step must still reach the CUDA kernels."""
    torch._dynamo.reset()
    compiled = torch.compile(model["step"], backend=backend, fullgraph=True, dynamic=False)
    for seed in (8, 9):
        x = P.make_activation(K0, seed=seed)
        out = compiled(x.cuda())
        torch.cuda.synchronize()
        _check(model, x, out, f"torch.compile[{backend}] seed {seed}")


def test_reference_modules_update_dec_config(model):
    """DECLinear.update_dec_config (DECLinear.py:45-53) re-points a layer at another context and k_chunk."""
    plugin = model["plugin"]
    rows2 = torch.zeros(1024, dtype=torch.int32, device="cuda")
    acts2 = torch.zeros(1024, dtype=torch.float16, device="cuda")
    ctx2 = plugin.create_dec_context(4, rows2, acts2)
    l0 = model["l0"]
    l0.update_dec_config(ctx2, 8)
    x = P.make_activation(K0, seed=11)
    y = l0(x.cuda())
    torch.cuda.synchronize()
    r, a, _ = P.expected_selection(x, l0.thresholds, 8, "fp16")
    assert np.array_equal(rows2[:16].cpu().numpy(), r)
    ref = ofw.layer_output(model["Lb"]["w_hat"], P.to_np(x), None,
                           ofw.dec_delta(P.to_np(x), r, l0.q_residual.numpy(), P.to_np(l0.scales), a))
    ma, rl = P.errors(y, ref)
    assert ma <= 1e-2 and rl <= 1e-3
    l0.update_dec_config(model["ctx"], KC)
