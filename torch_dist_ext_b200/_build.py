"""In-tree build of the native extension for sm_100a.

The reference builds through setuptools -> cmake.py -> CMakeLists.txt (setup.py:15-26,
cmake.py:52-115, CMakeLists.txt:1-38) and compiles for whatever architecture nvcc defaults to.
Here one ninja file is generated and run: device code is compiled by nvcc for exactly
``sm_100a`` (the ``a`` features - tcgen05, TMEM, multimem - are required), host-only and
binding code by g++, and everything is linked into ``torch_dist_ext_b200/_C.so`` next to the
Python sources so that the library is found without installation.

Usage::

    python -m torch_dist_ext_b200._build            # build if out of date
    python -m torch_dist_ext_b200._build --force    # rebuild everything
    python -m torch_dist_ext_b200._build --bounds   # also the range-checking flavour (TDX_BOUNDS=1 loads it)
    python -m torch_dist_ext_b200._build --trace    # also the tracing flavour (TDX_TRACE=1 loads it)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR.parent / "build" / "tdx"
LIB_PATH = PKG_DIR / "_C.so"
# Checked flavour: the fused all-reduce kernels and their launcher compiled with -DTDX_BOUNDS (every
# store into a symmetric allocation is range-checked, see csrc/include/tdx/sync.cuh), everything else
# shared with the release library. Loaded instead of _C.so when TDX_BOUNDS=1.
CHECKED_LIB_PATH = PKG_DIR / "_C_bounds.so"
# Tracing flavour: the same units compiled with -DTDX_TRACE (phase time stamps per block, see
# csrc/include/tdx/comm.h: TraceSlot). Loaded instead of _C.so when TDX_TRACE=1.
TRACED_LIB_PATH = PKG_DIR / "_C_trace.so"
FLAVOURS = {"bounds": ("-DTDX_BOUNDS", CHECKED_LIB_PATH), "trace": ("-DTDX_TRACE", TRACED_LIB_PATH)}
UNIT_TEST_SRC = PKG_DIR.parent / "tests" / "cpp" / "unit_test.cu"
UNIT_TEST_BIN = PKG_DIR.parent / "tests" / "cpp" / "unit_test.bin"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = NVCC_ARCH + [
    "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default", "--threads", "2",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]

# (source, object suffix, extra defines); device sources compiled by nvcc
DTYPES = {0: "f32", 1: "f16", 2: "bf16"}


def _device_units():
    units = []
    for code, name in DTYPES.items():
        for emu in (0, 1):
            units.append(("ar_fusion_inst.cu", f"ar_inst_{name}{'_emu' if emu else ''}",
                          [f"-DTDX_INST_DTYPE={code}", f"-DTDX_INST_EMU={emu}"]))
    for n in (0, 2, 4, 8):
        units.append(("gemm_fused.cu", f"gemm_fused_n{n}", [f"-DTDX_FUSED_N={n}"]))
    for src in sorted(CSRC.glob("*.cu")):
        if src.name in ("ar_fusion_inst.cu", "gemm_fused.cu"):
            continue
        units.append((src.name, src.stem, []))
    return units


def _host_units():
    """(source, needs_torch)"""
    out = []
    for src in sorted(CSRC.glob("*.cpp")):
        text = src.read_text()
        out.append((src.name, "torch/" in text or "tdx/bindings.h" in text or "ATen/" in text))
    return out


def _cuda_home() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and Path(cand, "bin", "nvcc").exists():
            return cand
    nvcc = shutil.which("nvcc")
    if nvcc:
        return str(Path(nvcc).resolve().parent.parent)
    raise RuntimeError("nvcc not found: set CUDA_HOME")


def _torch_flags():
    import torch
    from torch.utils import cpp_extension

    inc = [f"-isystem{p}" for p in cpp_extension.include_paths()]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    lib_dir = str(Path(torch.__file__).resolve().parent / "lib")
    return inc + [f"-D_GLIBCXX_USE_CXX11_ABI={abi}"], lib_dir, abi


def write_ninja() -> Path:
    cuda = _cuda_home()
    torch_inc, torch_lib, abi = _torch_flags()
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    inc = f"-I{CSRC / 'include'}"
    py_inc = subprocess.check_output(
        [sys.executable, "-c", "import sysconfig;print(sysconfig.get_paths()['include'])"], text=True).strip()
    lines = [
        "ninja_required_version = 1.3",
        f"nvcc = {cuda}/bin/nvcc",
        "cxx = g++",
        f"nvflags = {' '.join(NVCC_FLAGS)} {inc} -Xcompiler -D_GLIBCXX_USE_CXX11_ABI={abi}",
        f"cxxflags = {' '.join(CXX_FLAGS)} {inc} -isystem{cuda}/include -D_GLIBCXX_USE_CXX11_ABI={abi}",
        f"torchflags = {' '.join(torch_inc)} -isystem{py_inc}",
        "rule nvcc",
        "  command = $nvcc $nvflags $defs -MD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = NVCC $out",
        "rule cxx",
        "  command = $cxx $cxxflags $extra -MD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = CXX $out",
        "rule link",
        # linked under a temporary name and renamed, so that a process that loads (or a tool that copies) the library
        # while a rebuild runs never sees a partly written file
        "  command = $cxx -shared -o $out.tmp $in $ldflags && mv -f $out.tmp $out",
        "  description = LINK $out",
    ]
    objs = []
    for src, stem, defs in _device_units():
        obj = f"{stem}.o"
        objs.append(obj)
        lines += [f"build {obj}: nvcc {CSRC / src}", f"  defs = {' '.join(defs)}"]
    for src, needs_torch in _host_units():
        obj = f"{Path(src).stem}.host.o"
        objs.append(obj)
        lines += [f"build {obj}: cxx {CSRC / src}", f"  extra = {'$torchflags' if needs_torch else ''}"]
    ld = [
        f"-L{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda",
        f"-L{cuda}/lib64", "-lcudart", "-ldl", "-lpthread",
        f"-Wl,-rpath,{torch_lib}", "-Wl,--no-as-needed",
    ]
    lines += [f"build {LIB_PATH}: link {' '.join(objs)}", f"  ldflags = {' '.join(ld)}"]
    for flavour, (define, lib_path) in FLAVOURS.items():
        flavour_objs = []
        # the tracing flavour instruments the real launches only; the single-GPU emulation is shared
        # (and, in the tracing flavour, the prompt attention kernel with its per-role clock stamps)
        own_unit = (lambda stem: (stem.startswith("ar_inst_") and not (flavour == "trace" and stem.endswith("_emu")))
                    or (flavour == "trace" and stem == "attention_prefill_tc"))
        for obj in objs:
            if own_unit(obj[:-2]):
                flavour_objs.append(obj.replace(".o", f".{flavour}.o", 1))
            elif obj == "ar_fusion_launch.host.o":
                flavour_objs.append(f"ar_fusion_launch.{flavour}.host.o")
            else:
                flavour_objs.append(obj)
        for src, stem, defs in _device_units():
            if own_unit(stem):
                lines += [f"build {stem}.{flavour}.o: nvcc {CSRC / src}", f"  defs = {' '.join(defs)} {define}"]
        lines += [f"build ar_fusion_launch.{flavour}.host.o: cxx {CSRC / 'ar_fusion_launch.cpp'}", f"  extra = {define}"]
        lines += [f"build {lib_path}: link {' '.join(flavour_objs)}", f"  ldflags = {' '.join(ld)}"]
    # Standalone C++ harness (no PyTorch): the kernels, the launcher and the workspace manager only.
    core = [o for o in objs if o.startswith("ar_inst_") or o in ("workspace.o", "ar_fusion_launch.host.o", "fd_channel.host.o")]
    lines += [
        "rule nvlink_exe",
        "  command = $nvcc $nvflags -o $out.tmp $in -lcudart && mv -f $out.tmp $out",
        "  description = NVCC-LINK $out",
        f"build unit_test.o: nvcc {UNIT_TEST_SRC}",
        "  defs = ",
        f"build {UNIT_TEST_BIN}: nvlink_exe unit_test.o {' '.join(core)}",
        f"default {LIB_PATH} {UNIT_TEST_BIN}",
        "",
    ]
    path = BUILD_DIR / "build.ninja"
    text = "\n".join(lines)
    if not path.exists() or path.read_text() != text:
        path.write_text(text)
    return path


def build(force: bool = False, verbose: bool = False, checked: bool = False, traced: bool = False) -> Path:
    """Compile (if needed) and return the path of the extension library. ``checked`` also builds the
    range-checking flavour ``_C_bounds.so``, ``traced`` the tracing flavour ``_C_trace.so``."""
    write_ninja()
    if force:
        subprocess.run(["ninja", "-C", str(BUILD_DIR), "-t", "clean"], check=False,
                       stdout=subprocess.DEVNULL)
    cmd = ["ninja", "-C", str(BUILD_DIR)] + (["-v"] if verbose else [])
    if checked or traced:
        cmd += [str(LIB_PATH), str(UNIT_TEST_BIN)] + ([str(CHECKED_LIB_PATH)] if checked else []) + ([str(TRACED_LIB_PATH)] if traced else [])
    jobs = os.environ.get("TDX_BUILD_JOBS")
    if jobs:
        cmd += ["-j", jobs]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("native build failed:\n" + res.stdout[-8000:])
    if verbose:
        print(res.stdout)
    return CHECKED_LIB_PATH if checked else TRACED_LIB_PATH if traced else LIB_PATH


def clean() -> None:
    """Remove build products (what the reference's `setup.py clean` does via .gitignore parsing)."""
    shutil.rmtree(BUILD_DIR, ignore_errors=True)
    for lib in (LIB_PATH, CHECKED_LIB_PATH, TRACED_LIB_PATH):
        if lib.exists():
            lib.unlink()


if __name__ == "__main__":
    if "--clean" in sys.argv:
        clean()
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--bounds" in sys.argv,
                    traced="--trace" in sys.argv))
