"""Builds ``libpjx_attention.so`` in-tree with nvcc for sm_100a.

Run as ``python -m probjax_b200.build`` (add ``--force`` to rebuild, ``-v`` for
ptxas resource usage).  The library is rebuilt only when a source is newer than
it.  nvcc cross-compiles, so no GPU is needed to build.

``--what-if N --output PATH`` builds a second library whose tcgen05 forward kernel is compiled with
``-DPJX_EXP_VARIANT=N`` (timing experiments that remove one phase of the softmax loop: 9 no
exponentials, 11 no P store, 12 no softmax work at all, 13 no row maximum; 1-3 a share of the
exponentials on the FMA pipe); load it with ``PJX_ATTENTION_LIB=PATH``.  Variants 9-13 compute wrong
results on purpose and exist only to be timed.  ``--probe`` builds ``build/probe_mma_rate``, a
stand-alone program that times tcgen05.mma issue sequences.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libpjx_attention.so"

SOURCES = [
    "pjx_api.cu",
    "attn_fwd_generic.cu",
    "attn_bwd_generic.cu",
    "attn_bwd_sm100.cu",
    "attn_fwd_sm100.cu",
    "attn_decode.cu",
    "attn_decode_latent.cu",
    "attn_decode_latent_sm100.cu",
    "kv_cache.cu",
    "rope.cu",
    "rmsnorm.cu",
    "gemm_sm100.cu",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; it is required to build the CUDA library")
    return exe


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")) + [Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    common = [
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-std=c++17", "-lineinfo",
        "-Xcompiler", "-fPIC",
        "--expt-relaxed-constexpr",
        "-I", str(INCLUDE),
    ]
    if verbose:
        common += ["-Xptxas", "-v"]
    nvcc = _nvcc()
    procs = []
    for src in SOURCES:
        obj = objdir / (Path(src).stem + ".o")
        cmd = [nvcc, *common, "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out:
            print(out)
        objs.append(str(obj))
    link = [nvcc, "-shared", "-o", str(LIB), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    return LIB


FFI_LIB = PKG / "libpjx_ffi.so"


def jax_include_dir():
    """jaxlib's XLA FFI header directory, or None when jax is not installed."""
    try:
        import jax.ffi

        inc = jax.ffi.include_dir()
    except Exception:
        return None
    return inc if os.path.exists(os.path.join(inc, "xla", "ffi", "api", "ffi.h")) else None


def build_ffi(include_dir: str | None = None) -> Path | None:
    """Compiles ``csrc/ffi_shim.cc`` (the XLA FFI handlers over the C ABI) into ``libpjx_ffi.so``.
    Needs jaxlib's headers: returns None, building nothing, where they are absent."""
    include_dir = include_dir or jax_include_dir()
    if include_dir is None:
        return None
    build()
    cxx = shutil.which("g++") or "g++"
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    cmd = [cxx, "-std=c++17", "-O2", "-shared", "-fPIC", "-I", include_dir, "-I", str(INCLUDE), "-I", cuda_inc,
           str(CSRC / "ffi_shim.cc"), "-L", str(PKG), "-lpjx_attention", "-L", os.path.join(os.path.dirname(cuda_inc), "lib64"),
           "-lcudart", "-Wl,-rpath,$ORIGIN", "-o", str(FFI_LIB)]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"ffi shim build failed:\n{res.stdout}")
    return FFI_LIB


def build_what_if(variant: int, output: Path) -> Path:
    """The library with ``attn_fwd_sm100.cu`` compiled at ``-DPJX_EXP_VARIANT=variant``, linked with
    the regular objects of every other source."""
    build()
    objdir = PKG / "build"
    nvcc = _nvcc()
    obj = objdir / f"attn_fwd_sm100_what_if_{variant}.o"
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
           "--expt-relaxed-constexpr", "-I", str(INCLUDE), f"-DPJX_EXP_VARIANT={variant}", "-c",
           str(CSRC / "attn_fwd_sm100.cu"), "-o", str(obj)]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{res.stdout}")
    objs = [str(objdir / (Path(s).stem + ".o")) for s in SOURCES if s != "attn_fwd_sm100.cu"] + [str(obj)]
    res = subprocess.run([nvcc, "-shared", "-o", str(output), *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    return output


def build_probe() -> Path:
    """``csrc/probe_mma_rate.cu`` as the program ``build/probe_mma_rate`` (tcgen05.mma issue rates)."""
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    exe = objdir / "probe_mma_rate"
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-I", str(INCLUDE),
           str(CSRC / "probe_mma_rate.cu"), "-o", str(exe), "-lcuda"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{res.stdout}")
    return exe


if __name__ == "__main__":
    if "--probe" in sys.argv:
        print(build_probe())
        sys.exit(0)
    if "--what-if" in sys.argv:
        out = Path(sys.argv[sys.argv.index("--output") + 1]) if "--output" in sys.argv else PKG / "libpjx_what_if.so"
        print(build_what_if(int(sys.argv[sys.argv.index("--what-if") + 1]), out))
        sys.exit(0)
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    if "--ffi" in sys.argv:
        print(build_ffi() or "jaxlib headers not found: the FFI shim was not built")
