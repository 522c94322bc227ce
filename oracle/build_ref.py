"""Build the reference's own CUDA extension as a GPU-side cross-check (test infrastructure only).

    python oracle/build_ref.py [/path/to/DecDEC]

Compiles decdec_extension/{bindings.cpp, dec_context.cu, dec_config.cu, decdec.cu, dec.cu, sqllm.cu,
lutgemm.cu, anyprec.cu} of a reference checkout WHERE THEY LIE, unmodified, with the flags of the
reference's decdec_extension/setup.py:14-30 and one more code generation target (sm_100, which that
list does not name), into oracle/_ref/decdec_ref<EXT_SUFFIX>: the same pybind module under another name
(TORCH_EXTENSION_NAME=decdec_ref), so that a test process can load it beside this repository's
`decdec_ext`.  Objects and the module go to oracle/_ref/ only; no reference source is copied.

It also places the four small Python consumers of the binding (end-to-end/plugin.py, DECLinear.py,
APLinear.py, LUTGEMMLinear.py) under oracle/_ref/ref_modules/ so that a test on a machine without the
checkout can import them unchanged on top of this repository's `decdec_ext`.  oracle/_ref/ is not
tracked.

Nothing of the product imports the result: only tests/ (marked gpu) compare against it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
SOURCES = ["bindings.cpp", "dec_context.cu", "dec_config.cu", "decdec.cu", "dec.cu", "sqllm.cu", "lutgemm.cu", "anyprec.cu"]
CONSUMERS = ["plugin.py", "DECLinear.py", "APLinear.py", "LUTGEMMLinear.py"]
NAME = "decdec_ref"
# setup.py:16-24 of the reference, plus the one target its list lacks
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr",
              "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
              "-U__CUDA_NO_HALF2_OPERATORS__", "-U__CUDA_NO_HALF2_CONVERSIONS__",
              "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
              "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__",
              "-gencode=arch=compute_100,code=sm_100"]


def module_path() -> Path:
    return OUT / f"{NAME}{sysconfig.get_config_var('EXT_SUFFIX')}"


def build(ref_root: str, force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    src_dir = Path(ref_root) / "decdec_extension"
    if not src_dir.is_dir():
        raise FileNotFoundError(f"no decdec_extension under {ref_root}")
    OUT.mkdir(exist_ok=True)
    objdir = OUT / "obj"
    objdir.mkdir(exist_ok=True)
    try:
        inc = cpp_extension.include_paths("cuda")
    except TypeError:
        inc = cpp_extension.include_paths(cuda=True)
    common = [f"-I{p}" for p in inc] + [f"-I{sysconfig.get_paths()['include']}",
              f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    jobs = []
    objs = []
    for s in SOURCES:
        src = src_dir / s
        obj = objdir / (s.rsplit(".", 1)[0] + ".o")
        objs.append(str(obj))
        if not force and obj.exists() and obj.stat().st_mtime > src.stat().st_mtime:
            continue
        if s.endswith(".cu"):
            cmd = [NVCC, *NVCC_FLAGS, *common, "-Xcompiler", "-fPIC", "-c", str(src), "-o", str(obj)]
        else:
            cmd = ["g++", "-O3", "-DENABLE_BF16", "-std=c++17", "-fPIC", *common, "-c", str(src), "-o", str(obj)]
        jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        (OUT / "build.log").open("a").write(" ".join(cmd) + "\n" + r.stdout + "\n")
        if r.returncode != 0:
            raise RuntimeError(f"failed: {' '.join(cmd[:3])} ... {cmd[-1]}\n{r.stdout[-4000:]}")

    with ThreadPoolExecutor(max_workers=int(os.environ.get("JOBS", "8"))) as ex:
        list(ex.map(run, jobs))
    out = module_path()
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    if force or jobs or not out.exists():
        run(["g++", "-shared", "-o", str(out), *objs, f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
             "-ltorch_cuda", "-ltorch", "-ltorch_python", "-L/usr/local/cuda/lib64", "-lcudart",
             f"-Wl,-rpath,{torch_lib}"])
    mods = OUT / "ref_modules"
    mods.mkdir(exist_ok=True)
    for f in CONSUMERS:
        shutil.copyfile(Path(ref_root) / "end-to-end" / f, mods / f)
    return out


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DECDEC_REFERENCE", "")
    if not root:
        sys.exit("usage: python oracle/build_ref.py /path/to/DecDEC")
    print(build(root, force="--force" in sys.argv))
