"""In-tree build of the native code for sm_100a.

`python -m gpu_ipc_example_b200.build` writes a ninja file under
`gpu_ipc_example_b200/build/` and runs it.  Products (all inside the package so
that they travel with a snapshot of the source tree):

* `_C.so`            torch extension: custom ops + communicator bindings
* `libb200ipc.so`    the library without any torch dependency (C++ API + C entry points)
* `bin/main`         the benchmark / verification CLI
* `bin/list_devices` prints the GPUs and their peer-access matrix
* `libb200ipc_emu.so` CPU emulator of the wire protocols (no CUDA needed)

Every CUDA unit is compiled with `-gencode arch=compute_100a,code=sm_100a -lineinfo`.
Plays the role of the reference's Makefile (Makefile:1-42), which builds one
`main` binary ahead-of-time for one Intel GPU architecture.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "build"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

LL_OPS = ["ArParallel", "ArSequential", "ArRing", "ArBisect", "ArOneShot", "AgRing", "AgDirect", "RsParallel"]
LL_TYPES = {"f16": "__half", "bf16": "__nv_bfloat16"}

ARCH = "-gencode arch=compute_100a,code=sm_100a"


def _torch_flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-isystem {p}" for p in ce.include_paths(device_type="cuda")]
    inc.append(f"-isystem {sysconfig.get_paths()['include']}")
    lib_dir = Path(torch.__file__).parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    libs = [f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-ltorch_python"]
    return " ".join(inc), " ".join(defs), " ".join(libs), abi


def ninja_text(with_torch: bool = True) -> str:
    cuda_inc = f"-I{CUDA_HOME}/include"
    cuda_lib = f"-L{CUDA_HOME}/lib64 -Wl,-rpath,{CUDA_HOME}/lib64 -lcudart -ldl"
    abi_def = ""
    torch_inc = torch_defs = torch_libs = ""
    if with_torch:
        torch_inc, torch_defs, torch_libs, abi = _torch_flags()
        abi_def = f"-D_GLIBCXX_USE_CXX11_ABI={abi}"
        # libcudart shipped with torch must be the one resolved at run time inside python
    lines = []
    w = lines.append
    w("ninja_required_version = 1.5")
    w(f"builddir = {BUILD}")
    w(f"nvcc = {CUDA_HOME}/bin/nvcc")
    w("cxx = g++")
    w(f"cuflags = {ARCH} -lineinfo -O3 -std=c++17 --expt-relaxed-constexpr -Xcompiler -fPIC {abi_def} {cuda_inc}")
    w(f"cxxflags = -O2 -std=c++17 -fPIC -Wall -Wno-unknown-pragmas {abi_def} {cuda_inc}")
    w("rule cu")
    w("  command = $nvcc $cuflags $extra -MD -MF $out.d -c $in -o $out")
    w("  depfile = $out.d")
    w("  deps = gcc")
    w("  description = NVCC $out")
    w("rule cc")
    w("  command = $cxx $cxxflags $extra -MMD -MF $out.d -c $in -o $out")
    w("  depfile = $out.d")
    w("  deps = gcc")
    w("  description = CXX $out")
    w("rule link_so")
    w("  command = $cxx -shared -o $out $in $libs")
    w("  description = LINK $out")
    w("rule link_exe")
    w("  command = $cxx -o $out $in $libs")
    w("  description = LINK $out")

    core_objs = []

    def cc(src: str, extra: str = "") -> str:
        obj = f"$builddir/{src.replace('/', '_')}.o"
        w(f"build {obj}: cc {CSRC / src}")
        if extra:
            w(f"  extra = {extra}")
        return obj

    def cu(src: str, tag: str = "", extra: str = "") -> str:
        obj = f"$builddir/{src.replace('/', '_')}{tag}.o"
        w(f"build {obj}: cu {CSRC / src}")
        if extra:
            w(f"  extra = {extra}")
        return obj

    core_objs.append(cc("common/cu_driver.cpp"))
    core_objs.append(cc("bootstrap/unix_mesh.cpp"))
    core_objs.append(cc("mem/symm_heap.cpp"))
    core_objs.append(cc("mem/device_registry.cpp"))
    core_objs.append(cc("coll/comm.cpp"))
    core_objs.append(cc("coll/oracle.cpp"))
    for op in LL_OPS:
        for tag, ty in LL_TYPES.items():
            core_objs.append(cu("coll/ll_inst.cu", f".{op}.{tag}", f"-DB200_LL_OP={op} -DB200_LL_T={ty}"))
    core_objs.append(cu("coll/ll_table.cu"))
    core_objs.append(cu("coll/bulk_inst.cu"))
    core_objs.append(cu("fused/fused_ops.cu"))
    core_objs.append(cu("capi/no_alloc.cu"))
    core_objs.append(cu("fused/gemm_ar.cu"))
    core_objs.append(cu("model/decode_ops.cu"))

    lib = f"{PKG}/libb200ipc.so"
    w(f"build {lib}: link_so {' '.join(core_objs)}")
    w(f"  libs = {cuda_lib} -lpthread")

    emu_objs = [cc("emu/emulator.cpp")]
    emu = f"{PKG}/libb200ipc_emu.so"
    w(f"build {emu}: link_so {' '.join(emu_objs)}")
    w("  libs = -lpthread -lrt")

    main_obj = cc("cli/main.cpp")
    w(f"build {PKG}/bin/main: link_exe {main_obj} | {lib}")
    w(f"  libs = -L{PKG} '-Wl,-rpath,$$ORIGIN/..' -lb200ipc {cuda_lib} -lpthread")
    ld_obj = cc("cli/list_devices.cpp")
    w(f"build {PKG}/bin/list_devices: link_exe {ld_obj} | {lib}")
    w(f"  libs = -L{PKG} '-Wl,-rpath,$$ORIGIN/..' -lb200ipc {cuda_lib} -lpthread")

    targets = [lib, emu, f"{PKG}/bin/main", f"{PKG}/bin/list_devices"]
    if with_torch:
        bind = f"$builddir/torch_bindings.o"
        w(f"build {bind}: cc {CSRC / 'torch/bindings.cpp'}")
        w(f"  extra = {torch_inc} {torch_defs}")
        ext = f"{PKG}/_C.so"
        w(f"build {ext}: link_so {bind} | {lib}")
        w(f"  libs = -L{PKG} '-Wl,-rpath,$$ORIGIN' -lb200ipc {torch_libs} {cuda_lib}")
        targets.append(ext)
    w(f"default {' '.join(targets)}")
    return "\n".join(lines) + "\n"


def build(with_torch: bool = True, verbose: bool = False, jobs: int | None = None) -> None:
    BUILD.mkdir(exist_ok=True)
    (PKG / "bin").mkdir(exist_ok=True)
    text = ninja_text(with_torch)
    nf = BUILD / "build.ninja"
    if not nf.exists() or nf.read_text() != text:
        nf.write_text(text)
    ninja = shutil.which("ninja") or str(Path(sys.executable).parent / "ninja")
    cmd = [ninja, "-f", str(nf)]
    if jobs:
        cmd += ["-j", str(jobs)]
    if verbose:
        cmd.append("-v")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout[-20000:])
        raise RuntimeError("native build failed")
    if verbose:
        print(proc.stdout)


def cuda_units():
    """(source, extra flags) of every CUDA translation unit of the library."""
    units = [("coll/ll_inst.cu", f"-DB200_LL_OP={op} -DB200_LL_T={ty}") for op in LL_OPS for ty in LL_TYPES.values()]
    units += [(src, "") for src in ("coll/bulk_inst.cu", "fused/fused_ops.cu", "fused/gemm_ar.cu", "model/decode_ops.cu",
                                    "capi/no_alloc.cu")]
    return units


def ptxas_table() -> str:
    """Compiles every CUDA unit with `-Xptxas -v` (no GPU needed) and returns a markdown table of what the
    compiler reports per kernel: registers, stack frame, spill stores / loads, static shared memory."""
    import re

    rows = []
    for src, extra in cuda_units():
        cmd = (f"{CUDA_HOME}/bin/nvcc {ARCH} -lineinfo -O3 -std=c++17 --expt-relaxed-constexpr -Xptxas -v {extra} "
               f"-c {CSRC / src} -o /dev/null")
        proc = subprocess.run(cmd, shell=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            raise RuntimeError(proc.stdout[-4000:])
        text = subprocess.run(["c++filt"], input=proc.stdout, stdout=subprocess.PIPE, text=True).stdout
        name, frame = None, ("0", "0", "0")
        for line in text.splitlines():
            m = re.search(r"Compiling entry function '(.*)' for", line)
            if m:
                name = m.group(1)
                continue
            m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
            if m:
                frame = m.groups()
                continue
            m = re.search(r"Used (\d+) registers(?:, used \d+ barriers)?(?:, (\d+) bytes smem)?", line)
            if m and name:
                short = name.replace("void ", "").replace("b200ipc::", "").replace("(anonymous namespace)::", "")
                depth = 0  # drop the trailing parameter list
                for i in range(len(short) - 1, -1, -1):
                    depth += (short[i] == ")") - (short[i] == "(")
                    if depth == 0:
                        short = short[:i]
                        break
                rows.append((short, m.group(1), frame[0], frame[1], frame[2], m.group(2) or "0"))
                name = None
    out = ["| kernel | registers | stack B | spill st B | spill ld B | static smem B |", "|---|---|---|---|---|---|"]
    out += ["| `" + r[0] + "` | " + " | ".join(r[1:]) + " |" for r in rows]
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    if "--ptxas-table" in sys.argv:
        print(ptxas_table())
        sys.exit(0)
    build(with_torch="--no-torch" not in sys.argv, verbose="-v" in sys.argv)
    print("built:", ", ".join(sorted(p.name for p in PKG.glob("*.so"))))
