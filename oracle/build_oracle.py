"""Build recipes for the CPU checkers (TEST INFRASTRUCTURE ONLY).

* ``build_oracle_c()`` compiles ``oracle_c.c`` (this repository's own C
  restatement) into ``oracle/_build/liboracle.so``.
* ``build_ref()`` compiles the reference project's CPU retrieval backend
  (``ucm/sparse/gsa_on_device/csrc/cuda/hash_retrieval/cpy/hash_retrieval_backend.cpp``)
  straight from the reference checkout into ``oracle/_ref/``; no reference
  source is copied.  It is skipped when the checkout is not present (the
  prebuilt module, if any, is used as is).

* ``build_ref_cuda()`` compiles the reference project's CUDA Hamming-score
  extension (``.../csrc/cuda/ham_dist/paged_ham_dist_mla.cu`` + ``cpy/hamming.cpp``,
  unmodified, for sm_100) with ``torch.utils.cpp_extension`` into
  ``oracle/_ref/hamming_cuda/``: the GPU-side checker and the "reference kernel
  recompiled for B200" timing leg.  About two minutes of nvcc.

* ``build_ref_esa()`` compiles the reference project's ESA float-retrieval backend
  (``ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp``, unmodified) into ``oracle/_ref/``.  The
  file includes ``<numaif.h>``; where libnuma is not installed the stand-in header under
  ``oracle/shim/`` is put on the include path.

The reference checkout is found through the ``UCM_REFERENCE_ROOT`` environment variable (or the
``reference_root`` argument); without it only modules built earlier are used.

Run ``python oracle/build_oracle.py`` to build the CPU modules; add ``--cuda-ref`` for the CUDA one.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
REF_DIR = os.path.join(HERE, "_ref")
ORACLE_SO = os.path.join(BUILD_DIR, "liboracle.so")
REF_SRC_REL = "ucm/sparse/gsa_on_device/csrc/cuda/hash_retrieval/cpy/hash_retrieval_backend.cpp"


REF_ESA_SRC_REL = "ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp"
SHIM_DIR = os.path.join(HERE, "shim")


def _reference_root(arg: str | None) -> str:
    """The reference checkout: the argument, else $UCM_REFERENCE_ROOT, else a path that does not exist."""
    return arg or os.environ.get("UCM_REFERENCE_ROOT") or os.path.join(HERE, "_no_reference_checkout")


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_oracle_c(force: bool = False) -> str:
    src = os.path.join(HERE, "oracle_c.c")
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    os.makedirs(BUILD_DIR, exist_ok=True)
    cmd = ["gcc", "-O3", "-march=x86-64-v2", "-mpopcnt", "-fopenmp", "-shared", "-fPIC", "-std=c11",
           src, "-o", ORACLE_SO, "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def ref_module_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(REF_DIR, "hash_retrieval_backend" + suffix)


def build_ref(reference_root: str | None = None, force: bool = False) -> str | None:
    """Returns the module path, or None when neither source nor prebuilt module exists."""
    reference_root = _reference_root(reference_root)
    src = os.path.join(reference_root, REF_SRC_REL)
    out = ref_module_path()
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    if not force and _newer(out, src):
        return out
    import pybind11
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["g++", "-O3", "-march=x86-64-v2", "-mpopcnt", "-msse4.2", "-shared", "-fPIC", "-fopenmp",
           "-std=c++17", "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"],
           src, "-o", out, "-lpthread"]
    subprocess.check_call(cmd)
    return out


def ref_esa_module_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(REF_DIR, "retrieval_backend" + suffix)


def _have_system_numaif() -> bool:
    probe = subprocess.run(["g++", "-x", "c++", "-E", "-"], input=b"#include <numaif.h>\n", capture_output=True)
    return probe.returncode == 0


def build_ref_esa(reference_root: str | None = None, force: bool = False) -> str | None:
    """ESA float-retrieval backend of the reference, compiled unmodified.  Returns the module path, or None when
    neither source nor prebuilt module exists."""
    reference_root = _reference_root(reference_root)
    src = os.path.join(reference_root, REF_ESA_SRC_REL)
    out = ref_esa_module_path()
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    if not force and _newer(out, src):
        return out
    import pybind11
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["g++", "-O3", "-shared", "-fPIC", "-std=c++17", "-I" + pybind11.get_include(),
           "-I" + sysconfig.get_paths()["include"]]
    if not _have_system_numaif():
        cmd.append("-I" + SHIM_DIR)
    cmd += [src, "-o", out, "-lpthread"]
    subprocess.check_call(cmd)
    return out


def load_ref_esa():
    """Import the compiled ESA backend, or return None if it was never built."""
    path = ref_esa_module_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("retrieval_backend", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


REF_CUDA_DIR_REL = "ucm/sparse/gsa_on_device/csrc/cuda/ham_dist"
REF_CUDA_BUILD = os.path.join(REF_DIR, "hamming_cuda")
REF_CUDA_NAME = "ucm_ref_hamming"


# torch's extension builder defines these; the reference's own CMake build does not, and its kernel
# relies on the implicit __half conversions and operators.
_UNDEF_HALF = ["-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__"]


def ref_cuda_module_path() -> str:
    return os.path.join(REF_CUDA_BUILD, REF_CUDA_NAME + ".so")


def build_ref_cuda(reference_root: str | None = None, force: bool = False) -> str | None:
    """Returns the module path, or None when neither source nor prebuilt module exists."""
    reference_root = _reference_root(reference_root)
    src_dir = os.path.join(reference_root, REF_CUDA_DIR_REL)
    sources = [os.path.join(src_dir, "paged_ham_dist_mla.cu"), os.path.join(src_dir, "cpy", "hamming.cpp")]
    out = ref_cuda_module_path()
    if not all(os.path.exists(s) for s in sources):
        return out if os.path.exists(out) else None
    if not force and _newer(out, *sources):
        return out
    os.makedirs(REF_CUDA_BUILD, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils import cpp_extension
    cpp_extension.load(name=REF_CUDA_NAME, sources=sources, extra_include_paths=[src_dir],
                       extra_cflags=["-O3"], extra_cuda_cflags=["-O3", "--use_fast_math"] + _UNDEF_HALF,
                       build_directory=REF_CUDA_BUILD, is_python_module=True, verbose=False)
    return out if os.path.exists(out) else None


def load_ref_cuda():
    """Import the compiled reference CUDA extension (needs torch), or return None if it was never built."""
    path = ref_cuda_module_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(REF_CUDA_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_ref():
    """Import the compiled reference backend, or return None if it was never built."""
    path = ref_module_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("hash_retrieval_backend", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build_oracle_c(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    print(build_ref_esa(force="--force" in sys.argv))
    if "--cuda-ref" in sys.argv:
        print(build_ref_cuda(force="--force" in sys.argv))
