"""TEST INFRASTRUCTURE: compiles the reference's own CUDA ops, from the sources where they lie in the
mounted reference tree, into oracle/_ref/nanovllm_ref_ops.so (a pybind11 module with the reference's
`nanovllm.ops` functions). Nothing is copied into this repository; oracle/_ref/ is git-ignored and
only the built binary goes along to machines without the reference tree, where tests use it as a second checker
next to the CPU oracle (`load_reference_ops()` returns None when it is absent).

    python oracle/build_ref.py [<path of the reference tree>]

The reference builds this extension with setup.py (one CUDAExtension, -O3 -std=c++17, no fast-math,
setup.py:46-47,76-93); this recipe compiles the same eight sources with the same flags, for sm_100a.
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
MODULE = "nanovllm_ref_ops"
SO_PATH = os.path.join(OUT_DIR, MODULE + ".so")

SOURCES = [
    "csrc/ops.cpp", "csrc/pos_encoding_kernels.cu", "csrc/layernorm_kernels.cu", "csrc/activation_kernels.cu",
    "csrc/moe_align_block_size_kernels.cu", "csrc/moe_topk_softmax_kernels.cu", "csrc/store_kvcache_kernels.cu",
    "csrc/custom_all_reduce_kernels.cu",
]


def build_reference_ops(ref_root: str = "/root/reference", force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    srcs = [os.path.join(ref_root, s) for s in SOURCES]
    for s in srcs:
        if not os.path.exists(s):
            raise FileNotFoundError(s)
    if not force and os.path.exists(SO_PATH) and all(os.path.getmtime(SO_PATH) >= os.path.getmtime(s) for s in srcs):
        return SO_PATH
    os.makedirs(OUT_DIR, exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}",
                                                           f"-I{os.path.join(ref_root, 'csrc')}"]
    defs = [f"-DTORCH_EXTENSION_NAME={MODULE}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")

    def compile_one(src: str) -> str:
        obj = os.path.join(OUT_DIR, os.path.basename(src).rsplit(".", 1)[0] + ".o")
        if src.endswith(".cu"):
            cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
                   "--expt-relaxed-constexpr", *defs, *inc, "-c", src, "-o", obj]
        else:
            cmd = ["g++", "-O3", "-std=c++17", "-fPIC", *defs, *inc, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compiling {src} failed:\n{r.stderr[-4000:]}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_lib = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64")
    cmd = ["g++", "-shared", "-o", SO_PATH, *objs, f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
           "-ltorch_cuda", "-ltorch", "-ltorch_python", f"-L{cuda_lib}", "-lcudart", f"-L{cuda_lib}/stubs",
           "-Wl,--no-as-needed", "-lcuda", f"-Wl,-rpath,{torch_lib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking {SO_PATH} failed:\n{r.stderr[-4000:]}")
    for o in objs:
        os.remove(o)
    return SO_PATH


def load_reference_ops():
    """The reference's compiled ops as a module, or None when they were not built (or cannot load here,
    e.g. without a CUDA driver)."""
    if not os.path.exists(SO_PATH):
        return None
    try:
        import torch  # noqa: F401  (its libraries must be loaded first)
        loader = importlib.machinery.ExtensionFileLoader(MODULE, SO_PATH)
        spec = importlib.util.spec_from_loader(MODULE, loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        return mod
    except Exception as e:  # noqa: BLE001
        print(f"[oracle] reference ops present but not loadable: {e}")
        return None


if __name__ == "__main__":
    print(build_reference_ops(sys.argv[1] if len(sys.argv) > 1 else "/root/reference", force=True))
