"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own Python functions
(SNU-ARC/DecDEC checked out at REF, the first argument) on small seeded inputs.

    python tests/golden/make_golden.py REF

Functions exercised (CPU torch, no GPU needed):
  decdec_setup/cheatsheet.py:_process_layer                      residual quantizer + packer
  decdec_setup/llm-awq/quantize/quantizer.py:pseudo_quantize_tensor   asymmetric group quantizer
  evaluation/evaltools.py:lutgemm_dequant, sqllm_dequant          dense weights of packed tensors
`evaltools.py` imports the CUDA extension and the lm-eval harness at module level; both are replaced
by empty stand-in modules for the import (none of their functions is called).
The reference cannot be imported on the GPU test machine, so the vectors are committed.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

if len(sys.argv) < 2:
    raise SystemExit("usage: python " + sys.argv[0] + " <path of the SNU-ARC/DecDEC checkout>")
REF = sys.argv[1]
OUT = os.path.dirname(os.path.abspath(__file__))


def load(path, name, stubs=()):
    for s in stubs:
        name_, _, attrs = s.partition(":")
        if name_ not in sys.modules:
            m = types.ModuleType(name_)
            m.__path__ = []
            sys.modules[name_] = m
        for a in filter(None, attrs.split(",")):
            setattr(sys.modules[name_], a, None)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    torch.manual_seed(0)
    rng = np.random.default_rng(0)

    # ---- residual quantizer / packer -------------------------------------------------------------
    cheat = load(os.path.join(REF, "decdec_setup", "cheatsheet.py"), "ref_cheatsheet")
    N, K = 64, 256

    class Layer(torch.nn.Module):
        def __init__(self, w):
            super().__init__()
            self.proj = torch.nn.Linear(K, N, bias=False, dtype=torch.float16)
            self.proj.weight.data = w

    w = (torch.randn(N, K) * 0.02).half()
    wq = (w.float() + torch.randn(N, K) * 0.002).half()          # stands for the fake-quantized weight
    per_layer, _, _ = cheat._process_layer((0, Layer(w), Layer(wq), False, False))
    cs = per_layer["proj"]["cheatsheet"].numpy()
    rs = per_layer["proj"]["reordered_scales"].numpy()
    np.savez(os.path.join(OUT, "cheatsheet.npz"), w=w.numpy(), wq=wq.numpy(), cheatsheet=cs, reordered_scales=rs)

    # ---- uniform quantizer ---------------------------------------------------------------------------
    sys.path.insert(0, os.path.join(REF, "decdec_setup", "llm-awq"))
    import quantize.quantizer as qz                                  # the reference package itself
    wu = (torch.randn(32, 512) * 0.02).float()
    for bits in (3, 4):
        wf, sc, zp = qz.pseudo_quantize_tensor(wu.clone(), n_bit=bits, zero_point=True, q_group_size=128, get_scale_zp=True)
        np.savez(os.path.join(OUT, f"uniform_b{bits}.npz"), w=wu.numpy(), w_fake=wf.numpy(), scales=sc.numpy(), zeros=zp.numpy())

    # ---- dense weights of packed tensors ----------------------------------------------------------------
    ev = load(os.path.join(REF, "evaluation", "evaltools.py"), "ref_evaltools",
              stubs=("decdec_ext", "lm_eval", "accelerate:init_empty_weights", "datasets:load_dataset"))
    Kb, Nb, bits, group = 256, 48, 3, 128
    binary = torch.from_numpy(rng.integers(-2**31, 2**31, size=(Kb // 32, bits, Nb), dtype=np.int64).astype(np.int32))
    alpha = (torch.rand(Kb // group, bits, Nb) * 0.01).half()
    q_bias = ((torch.rand(Kb // group, Nb) - 0.5) * 0.01).half()
    dense = ev.lutgemm_dequant(binary, alpha, q_bias, bits, group)
    np.savez(os.path.join(OUT, "lutgemm_dequant.npz"), binary=binary.numpy(), alpha=alpha.numpy(), q_bias=q_bias.numpy(),
             dense=dense.float().numpy(), group=group)
    for b in (3, 4):
        qw = torch.from_numpy(rng.integers(-2**31, 2**31, size=(Kb * b // 32, Nb), dtype=np.int64).astype(np.int32))
        lut = (torch.randn(Nb, 2 ** b) * 0.02).half()
        dense = ev.sqllm_dequant(qw, lut, b)
        np.savez(os.path.join(OUT, f"sqllm_dequant_b{b}.npz"), qweight=qw.numpy(), lut=lut.numpy(), dense=dense.float().numpy())
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
