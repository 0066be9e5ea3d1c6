"""In-tree build of the two native libraries.

* ``catch_b200/lib/libcatch_b200_device.so`` -- every ``csrc/device/*.cu`` file,
  compiled by nvcc for sm_100a only (CUDA runtime wrappers + all kernels, C ABI).
* ``catch_b200/_C*.so`` -- the host runtime, operator registrations, process
  group, TorchScript passes and Python bindings (``csrc/**/*.cpp``), compiled by
  g++ against libtorch and linked to the device library.

The reference builds three CMake libraries plus a setuptools stub
(setup.py:244-252, torch_mlu/csrc/CMakeLists.txt:186-204); here a generated
ninja file does the same job so that incremental rebuilds take seconds and the
outputs stay inside the source tree.

Usage: ``python -m catch_b200._build [--clean] [-v]``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "catch_b200"
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"
DEVICE_LIB = PKG / "lib" / "libcatch_b200_device.so"
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
HOST_LIB = PKG / f"_C{EXT_SUFFIX}"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# The system g++ (same libstdc++ ABI as libtorch).  $CXX is ignored on purpose:
# some images point it at a toolchain that links libstdc++ statically, which
# breaks iostreams inside a Python extension.
CXX = os.environ.get("CATCH_B200_CXX", "/usr/bin/g++")

# Build switches (environment), the counterpart of the reference's setup.py flags (setup.py:24-34,190-204):
#   DEBUG=1                    host code with -O0 -g and assertions, device code with -G left off (-lineinfo stays)
#   CATCH_B200_BUILD_ASAN=1    AddressSanitizer for the host libraries (host side only, like RUN_BUILD_ASAN_CHECK)
#   CATCH_B200_BUILD_UBSAN=1   UndefinedBehaviorSanitizer for the host libraries (reports are printed, execution goes on)
#   CATCH_B200_BUILD_TEST=0    skip the C++ test program
#   MAX_JOBS=n                 parallel compile jobs
DEBUG = os.environ.get("DEBUG", "0") not in ("0", "", "OFF", "off")
ASAN = os.environ.get("CATCH_B200_BUILD_ASAN", "0") not in ("0", "", "OFF", "off")
UBSAN = os.environ.get("CATCH_B200_BUILD_UBSAN", "0") not in ("0", "", "OFF", "off")
SANITIZE = (["-fsanitize=address"] if ASAN else []) + (["-fsanitize=signed-integer-overflow,shift,integer-divide-by-zero,bounds,alignment,float-cast-overflow,float-divide-by-zero,bool,enum,return,unreachable,vla-bound"] if UBSAN else [])
BUILD_TEST = os.environ.get("CATCH_B200_BUILD_TEST", "1") not in ("0", "OFF", "off")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
] + ([] if DEBUG else ["-DNDEBUG"])


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths()
    lib = [str(Path(torch.__file__).parent / "lib")]
    return inc, lib


def _nccl_paths():
    try:
        import nvidia.nccl as n  # type: ignore

        base = Path(n.__path__[0])
        return str(base / "include"), str(base / "lib")
    except Exception:
        return None, None


def device_sources():
    return sorted(CSRC.glob("device/*.cu"))


def host_sources():
    out = []
    for sub in ("runtime", "ops", "distributed", "jit", "python"):
        out += sorted((CSRC / sub).glob("*.cpp"))
    return out


def write_ninja(verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    (PKG / "lib").mkdir(exist_ok=True)
    inc, lib = _torch_paths()
    nccl_inc, nccl_lib = _nccl_paths()
    py_inc = sysconfig.get_paths()["include"]
    cxx_inc = " ".join(f"-isystem {p}" for p in inc + [py_inc] + ([nccl_inc] if nccl_inc else []))
    cxx_flags = (
        ("-O0 -g " if DEBUG else "-O2 -DNDEBUG ") + (" ".join(SANITIZE) + " -fno-omit-frame-pointer " if SANITIZE else "") +
        "-std=c++17 -fPIC -fvisibility=hidden -Wall -Wno-unused-variable -Wno-unused-function "
        "-Wno-sign-compare -Wno-unknown-pragmas -D_GLIBCXX_USE_CXX11_ABI=1 -DTORCH_EXTENSION_NAME=_C "
        "-DTORCH_API_INCLUDE_EXTENSION_H"
    )
    lines = [
        "ninja_required_version = 1.3",
        f"nvcc = {NVCC}",
        f"cxx = {CXX}",
        f"nvcc_flags = {' '.join(NVCC_FLAGS)} -I{CSRC}",
        f"cxx_flags = {cxx_flags} {cxx_inc} -I{CSRC}",
        "",
        "rule nvcc",
        "  command = $nvcc $nvcc_flags -MD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = NVCC $in",
        "rule cxx",
        "  command = $cxx $cxx_flags -MMD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = CXX $in",
        "rule link_device",
        "  command = $nvcc -shared -o $out $in -Xlinker -soname=libcatch_b200_device.so -lpthread -ldl",
        "  description = LINK $out",
        "rule link_host",
        "  command = $cxx -shared -o $out $in $ldflags",
        "  description = LINK $out",
        "",
    ]
    dev_objs = []
    for src in device_sources():
        obj = BUILD / "device" / (src.stem + ".o")
        dev_objs.append(obj)
        lines.append(f"build {obj}: nvcc {src}")
    lines.append(f"build {DEVICE_LIB}: link_device {' '.join(map(str, dev_objs))}")
    host_objs = []
    for src in host_sources():
        obj = BUILD / "host" / src.parent.name / (src.stem + ".o")
        host_objs.append(obj)
        lines.append(f"build {obj}: cxx {src}")
    ld = [f"-L{p}" for p in lib] + [
        "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
        f"-L{PKG / 'lib'}", "-lcatch_b200_device",
        "-Wl,-rpath,$$ORIGIN/lib", "-Wl,--no-as-needed",
    ] + SANITIZE
    for p in lib:
        ld.append(f"-Wl,-rpath,{p}")
    lines.append(f"build {HOST_LIB}: link_host {' '.join(map(str, host_objs))} | {DEVICE_LIB}")
    lines.append(f"  ldflags = {' '.join(ld)}")
    # C++ test program of the runtime (no Python): runtime objects + test main
    test_bin = PKG / "lib" / "b200_runtime_test"
    test_objs = []
    for src in sorted((CSRC / "test").glob("*.cpp")):
        obj = BUILD / "host" / "test" / (src.stem + ".o")
        test_objs.append(obj)
        lines.append(f"build {obj}: cxx {src}")
    if test_objs and BUILD_TEST:
        rt_objs = [o for o in host_objs if o.parent.name in ("runtime", "jit")]
        ld_test = [f"-L{p}" for p in lib] + ["-lc10", "-ltorch_cpu", "-ltorch", f"-L{PKG / 'lib'}", "-lcatch_b200_device",
                                             "-Wl,-rpath,'$$ORIGIN'", "-Wl,--no-as-needed", "-lpthread"] + SANITIZE
        for p in lib:
            ld_test.append(f"-Wl,-rpath,{p}")
        lines.insert(lines.index("rule link_host"), "rule link_exe")
        lines.insert(lines.index("rule link_host"), "  command = $cxx -o $out $in $ldflags")
        lines.insert(lines.index("rule link_host"), "  description = LINK $out")
        lines.append(f"build {test_bin}: link_exe {' '.join(map(str, test_objs + rt_objs))} | {DEVICE_LIB}")
        lines.append(f"  ldflags = {' '.join(ld_test)}")
        lines.append(f"default {DEVICE_LIB} {HOST_LIB} {test_bin}")
    else:
        lines.append(f"default {DEVICE_LIB} {HOST_LIB}")
    path = BUILD / "build.ninja"
    text = "\n".join(lines) + "\n"
    if not path.exists() or path.read_text() != text:
        path.write_text(text)
    return path


def build(verbose: bool = False, clean: bool = False, targets=()) -> None:
    if clean and BUILD.exists():
        shutil.rmtree(BUILD)
    write_ninja(verbose)
    jobs = os.environ.get("MAX_JOBS", str(os.cpu_count() or 4))
    cmd = ["ninja", "-C", str(BUILD), "-j", jobs]
    if verbose:
        cmd.append("-v")
    cmd += [str(t) for t in targets]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError("catch_b200 native build failed")
    if verbose:
        sys.stdout.write(proc.stdout)


def is_built() -> bool:
    return DEVICE_LIB.exists() and HOST_LIB.exists()


if __name__ == "__main__":
    build(verbose="-v" in sys.argv, clean="--clean" in sys.argv,
          targets=[DEVICE_LIB] if "--device-only" in sys.argv else ())
    print("built:", DEVICE_LIB, HOST_LIB)
