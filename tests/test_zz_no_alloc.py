"""GPU test of `decdec_lutgemm_gemv_noalloc`, the entry point for hosts that may not allocate device
memory at call time (an application that owns the whole device heap, a real-time loop).  It keeps its accumulator in a fixed array inside the library instead of a
cudaMalloc'd workspace.  The test calls it through the C ABI twice in a row and checks both results
against the regular `decdec_lutgemm_gemv` within the fp16 tolerance of the parity tests (max abs 1e-2,
rel L2 1e-3 against the oracle; the two entry points themselves must agree to output rounding).

Collected last on purpose (file name), so that a failure here cannot hide the other tests under -x.
"""
import numpy as np
import pytest
import torch

from oracle import forward as ofw
from tests import problems as P

pytestmark = pytest.mark.gpu


def _call(capi, name, x, y, L, bits, group):
    capi.call(name, x.data_ptr(), y.data_ptr(), L["qweight"].data_ptr(), L["alpha"].data_ptr(), L["q_bias"].data_ptr(),
              y.numel(), x.numel(), bits, group, capi.FP16, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("N,K", [(4096, 4096), (200, 1088)])   # TMA-pipelined shape and a ragged one
def test_noalloc_matches_regular_entry_point_twice(N, K):
    assert torch.cuda.is_available()
    from decdec_b200 import capi
    group = 128 if K % 128 == 0 else 32
    L = P.random_bcq_layer(N, K, 3, group, seed=17)
    Ld = {k: v.cuda() for k, v in L.items() if isinstance(v, torch.Tensor)}
    for rep, seed in enumerate((1, 2)):                       # two calls in a row share the static scratch
        x = P.make_activation(K, seed=seed)
        y0 = (torch.randn(1, 1, N, generator=torch.Generator().manual_seed(seed)) * 0.5).half()
        y_ref, y_new = y0.clone().cuda(), y0.clone().cuda()
        xd = x.cuda()
        _call(capi, "decdec_lutgemm_gemv", xd, y_ref, Ld, 3, group)
        _call(capi, "decdec_lutgemm_gemv_noalloc", xd, y_new, Ld, 3, group)
        torch.cuda.synchronize()
        ref = ofw.layer_output(L["w_hat"], P.to_np(x), P.to_np(y0))
        for name, y in (("regular", y_ref), ("noalloc", y_new)):
            ma, rl = P.errors(y, ref)
            assert ma <= 1e-2 and rl <= 1e-3, f"call {rep} {name}: max abs {ma:.3e}, rel L2 {rl:.3e}"
        # same kernel, same inputs: only the fp32 reduction order may differ -> one fp16 ulp at most
        assert (y_ref.float() - y_new.float()).abs().max().item() <= 2e-2


def test_noalloc_rejects_sizes_beyond_the_static_scratch():
    from decdec_b200 import capi
    with pytest.raises(capi.DecdecError, match="static scratch limit") as e:
        capi.call("decdec_lutgemm_gemv_noalloc", 16, 16, 16, 16, 16, 32768 + 128, 1024, 3, 128, capi.FP16, None)
    assert e.value.code == -2
