"""In-tree build of the native pieces (no GPU needed: nvcc cross-compiles for sm_100a).

    python -m feather_ops_b200._build          # build what is stale
    python -m feather_ops_b200._build --force  # rebuild everything

Products, all beside this file:
  libfeather_ops_b200.so  the torch-free C-ABI library (kernels + launchers declared in include/feather_ops_b200.h)
  _C.so                   the thin torch extension: registers `torch.ops.feather_ops.*` and forwards to the C ABI

The tile lookup header `csrc/feather_tiles_gen.h` is regenerated from `tiles.py` on every build.
"""

import argparse
import concurrent.futures
import importlib.util
import os
import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
ROOT = PKG.parent
OBJ = PKG / "build"
LIB = PKG / "libfeather_ops_b200.so"
EXT = PKG / "_C.so"
TILE_HEADER = CSRC / "feather_tiles_gen.h"

KERNEL_SOURCES = [
    "scaled_mm_sm100.cu",
    "convrot_quantize_sm100.cu",
    "int8_mm_sm100.cu",
    "conv3x3_sm100.cu",
    "selftest_sm100.cu",
]
NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
    "--expt-relaxed-constexpr",
]


def _load_tiles():
    spec = importlib.util.spec_from_file_location("_feather_b200_tiles", PKG / "tiles.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def write_tile_header() -> bool:
    """Regenerate the tile lookup header. Returns True if the file changed."""
    rendered = _load_tiles().render_header()
    if TILE_HEADER.exists() and TILE_HEADER.read_text() == rendered:
        return False
    TILE_HEADER.write_text(rendered)
    return True


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return found


def _stale(target: pathlib.Path, deps: list[pathlib.Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(dep.stat().st_mtime > stamp for dep in deps if dep.exists())


def _run(cmd: list[str], log: pathlib.Path | None = None) -> None:
    result = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(result.stdout + result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{result.stdout}\n{result.stderr}")


def build_kernels(force: bool = False) -> None:
    OBJ.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    sources = [CSRC / name for name in KERNEL_SOURCES if (CSRC / name).exists()]
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            jobs.append(([_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], OBJ / (src.stem + ".ptxas.log")))
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        for future in [pool.submit(_run, cmd, log) for cmd, log in jobs]:
            future.result()
    objects = [OBJ / (src.stem + ".o") for src in sources]
    if force or jobs or _stale(LIB, objects):
        _run([_nvcc(), "-shared", "-o", str(LIB), *[str(o) for o in objects], "-Xcompiler", "-fPIC", "-cudart", "static"])


def build_extension(force: bool = False) -> None:
    src = CSRC / "torch_ops.cpp"
    if not src.exists():
        return
    if not (force or _stale(EXT, [src, LIB, ROOT / "include" / "feather_ops_b200.h"])):
        return
    import torch

    torch_dir = pathlib.Path(torch.__file__).resolve().parent
    import sysconfig

    cmd = [
        "g++",
        "-O2",
        "-std=c++17",
        "-fPIC",
        "-shared",
        "-DTORCH_TARGET_VERSION=0x020A000000000000",
        "-DTORCH_STABLE_ONLY",
        "-DUSE_CUDA",
        "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch.compiled_with_cxx11_abi())),
        "-I",
        str(torch_dir / "include"),
        "-I",
        str(ROOT / "include"),
        "-I",
        sysconfig.get_paths()["include"],
        "-I",
        "/usr/local/cuda/include",
        str(src),
        "-o",
        str(EXT),
        "-L",
        str(PKG),
        "-lfeather_ops_b200",
        "-L",
        str(torch_dir / "lib"),
        "-ltorch",
        "-ltorch_cpu",
        "-ltorch_cuda",
        "-lc10",
        "-Wl,-rpath,$ORIGIN",
        "-Wl,-rpath," + str(torch_dir / "lib"),
    ]
    _run(cmd)


def build_all(force: bool = False) -> None:
    changed = write_tile_header()
    build_kernels(force or changed)
    build_extension(force)


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args()
    build_all(args.force)
    print(f"built {LIB.name}" + (f" and {EXT.name}" if EXT.exists() else ""))
    sys.exit(0)
