"""In-tree build of the native library (nvcc, sm_100a only).

`build_native()` compiles every `csrc/*.cu` into `leopard_b200/lib/libleopard_b200.so`.  nvcc cross-compiles
without a GPU, so this runs in the authoring container; the built `.so` travels to the GPU box with the repo
snapshot (it is git-ignored, not gpurun-ignored).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libleopard_b200.so"
OBJDIR = LIBDIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


# components: a library of its own for a subset of the sources (the full library contains every component)
COMPONENTS = {
    # decoder-only language models on the 32-bit residual-stream kernels, plus the tcgen05 GEMM that takes their large bf16 products
    "stream32": ("lp_host.cu", "lp_linear.cu", "lp_stream32.cu", "lp_seqmix.cu", "lp_winattn.cu", "lp_mingru.cu", "lp_mlstm.cu", "lp_moe.cu", "lp_gemm.cu",
                 "lp_gemm4.cu"),
}


def sources(component=None):
    if component is None:
        return sorted(CSRC.glob("*.cu"))
    return [CSRC / n for n in COMPONENTS[component]]


def _deps(component=None):
    return sources(component) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG.parent / "include" / "leopard_b200.h"]


def _paths(component=None):
    if component is None:
        return LIB, OBJDIR, LIBDIR / "build.sha256"
    return LIBDIR / f"libleopard_{component}.so", LIBDIR / f"obj_{component}", LIBDIR / f"build_{component}.sha256"


def is_current(component=None) -> bool:
    """True when the (component's) library exists and was built from the sources as they are now."""
    lib, _, stamp = _paths(component)
    return lib.exists() and stamp.exists() and stamp.read_text().strip() == _digest(_deps(component))


def build_native(force: bool = False, verbose: bool = False, component=None) -> Path:
    """Compile csrc/*.cu -> lib/libleopard_b200.so, or one component's sources -> lib/libleopard_<component>.so (skipped when the
    sources are unchanged).  Objects are written under a private name and renamed, so that two processes may build at once."""
    lib_path, objdir, stamp = _paths(component)
    LIBDIR.mkdir(exist_ok=True)
    objdir.mkdir(exist_ok=True)
    dig = _digest(_deps(component))
    if not force and is_current(component):
        return lib_path
    nvcc = _nvcc()
    tag = f".{os.getpid()}"

    def compile_one(src: Path):
        obj = objdir / (src.stem + tag + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        (objdir / (src.stem + ".ptxas.log")).write_text(r.stderr)
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources(component)))
    tmp_lib = lib_path.with_name(lib_path.name + tag)
    cmd = [nvcc, "-shared", "-o", str(tmp_lib), *map(str, objs), "-cudart", "static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    for o in objs:
        os.replace(o, o.with_name(o.name.replace(tag + ".o", ".o")))
    os.replace(tmp_lib, lib_path)
    stamp.write_text(dig)
    return lib_path


if __name__ == "__main__":
    comp = next((a for a in sys.argv[1:] if a in COMPONENTS), None)
    print(build_native(force="--force" in sys.argv, verbose="-v" in sys.argv, component=comp))
