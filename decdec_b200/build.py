"""Build the native parts in-tree.

  python -m decdec_b200.build            # libdecdec_b200.so (CUDA, C ABI) + decdec_ext torch shim
  python -m decdec_b200.build --lib      # only the CUDA library

Both products land inside the package directory so that they travel with a source snapshot.
The CUDA library is compiled for sm_100a only.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libdecdec_b200.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CU_SOURCES = ["host.cu", "k_dec.cu", "k_bcq.cu", "k_anyprec.cu", "k_sqllm.cu", "noalloc.cu", "tp_allreduce.cu"]


def _run(cmd, log=None):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.append(res.stdout)
    if res.returncode != 0:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + res.stdout)
        raise RuntimeError(f"command failed: {cmd[0]} ... {cmd[-1]}")
    return res.stdout


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_lib(verbose: bool = False, force: bool = False) -> Path:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG.parent / "include" / "decdec_b200.h"]
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    sources = [s for s in CU_SOURCES if (CSRC / s).exists()]
    jobs = []
    for src in sources:
        obj = objdir / (src.replace(".cu", ".o"))
        if force or _stale(obj, [CSRC / src] + headers):
            cmd = [NVCC, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-DNDEBUG", "-c", str(CSRC / src), "-o", str(obj)]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    logs = []
    with ThreadPoolExecutor(max_workers=min(6, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, logs), jobs))
    if verbose:
        print("\n".join(logs))
    objs = [str(objdir / s.replace(".cu", ".o")) for s in sources]
    if force or jobs or _stale(LIB, objs):
        _run([NVCC, *ARCH, "-shared", "-o", str(LIB), *objs, "-lcudart"])
    return LIB


def build_shim(force: bool = False) -> Path:
    """decdec_ext: pybind11/torch module with the reference's 17 functions (bindings.cpp:17-41)."""
    import torch
    from torch.utils import cpp_extension

    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    out = PKG / f"decdec_ext{suffix}"
    src = CSRC / "shim.cpp"
    if not force and not _stale(out, [src, PKG.parent / "include" / "decdec_b200.h"]):
        return out
    inc = cpp_extension.include_paths(device_type="cuda") if hasattr(cpp_extension, "include_paths") else []
    try:
        inc = cpp_extension.include_paths("cuda")
    except TypeError:
        inc = cpp_extension.include_paths(cuda=True)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=decdec_ext",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{p}" for p in inc], f"-I{sysconfig.get_paths()['include']}", f"-I{PKG.parent / 'include'}",
           str(src), "-o", str(out), f"-L{PKG}", "-ldecdec_b200", f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
           "-ltorch_cuda", "-ltorch", "-ltorch_python", "-L/usr/local/cuda/lib64", "-lcudart",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--lib", action="store_true", help="only build the CUDA library")
    ap.add_argument("--verbose", action="store_true", help="print ptxas resource usage")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    print(build_lib(a.verbose, a.force))
    if not a.lib:
        print(build_shim(a.force))


if __name__ == "__main__":
    main()
