"""In-tree build of the native libraries.

* ``libovb_cuda.so``  - sm_100a kernels (nvcc, C ABI, loaded with ctypes)
* ``_ovcore*.so``     - native core: graph IR, IR v11 reader/writer, passes, CPU reference
                        executor, runtime and scheduler (g++ + pybind11)
* ``libopenvino_b200_c.so`` - the same core behind the C API (no Python dependency)

Both are written next to the sources inside the package so that a checkout is
self-contained: nothing is installed into site-packages and no JIT cache is used.
Run ``python -m openvino_b200.build`` to (re)build; imports trigger a build only when
a library is missing or older than its sources.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = PKG / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout[-4000:], r.stderr[-8000:]))


def cuda_sources() -> list[Path]:
    return sorted((CSRC / "cuda").glob("*.cu"))


def build_cuda_debug(force: bool = False) -> Path:
    """The bounds-checking debug build of the kernels: ``lib/libovb_cuda_dbg.so`` (compiled with -DOVB_DEBUG_BOUNDS, objects
    under ``build/dbg``). Load it with ``OVB_CUDA_LIB``; see csrc/cuda/debug_bounds.cuh."""
    return build_cuda(force, False, ("-DOVB_DEBUG_BOUNDS",), "_dbg")


def build_cuda(force: bool = False, verbose: bool = False, extra_flags=(), suffix: str = "") -> Path:
    """Compile every .cu under csrc/cuda for sm_100a and link libovb_cuda.so."""
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    target = LIB / ("libovb_cuda%s.so" % suffix)
    obj_dir = OBJ / suffix.strip("_") if suffix else OBJ
    obj_dir.mkdir(exist_ok=True)
    srcs = cuda_sources()
    hdrs = sorted((CSRC / "cuda").glob("*.cuh")) + sorted((CSRC / "cuda").glob("*.h"))
    if not force and not _stale(target, srcs + hdrs):
        return target
    nvcc = _nvcc()

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        if force or _stale(obj, [src] + hdrs):
            # ptxas reports registers, stack frame and spills of every kernel; the report is kept next to the object
            # (build/<name>.ptxas.txt) so that a resource regression of a hot kernel shows up without a GPU
            cmd = [nvcc, "-Xptxas", "-v", *NVCC_FLAGS, *extra_flags, "-I", str(CSRC / "cuda"), "-c", str(src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout[-4000:], r.stderr[-8000:]))
            (obj_dir / (src.stem + ".ptxas.txt")).write_text(r.stderr)
            if verbose:
                print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    # only the C ABI is exported; everything else (C++ runtime templates, the static CUDA runtime) stays local
    vers = obj_dir / "ovb_cuda.map"
    vers.write_text("{ global: ovb_*; local: *; };\n")
    _run([nvcc, "-shared", "-o", str(target), *map(str, objs), "-cudart", "static", "-Xlinker", "--version-script=%s" % vers])
    return target


def core_sources() -> list[Path]:
    return sorted((CSRC / "core").glob("*.cpp"))


def build_core(force: bool = False) -> Path | None:
    """Compile the native core into a CPython extension module (pybind11)."""
    srcs = core_sources()
    if not srcs:
        return None
    import pybind11

    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    target = PKG / ("_ovcore" + ext)
    hdrs = sorted((CSRC / "core").glob("*.hpp")) + sorted((CSRC / "core").glob("*.h"))
    if not force and not _stale(target, srcs + hdrs):
        return target
    cxx = os.environ.get("CXX", "g++")
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(CSRC / "core")]

    def compile_one(src: Path) -> Path:
        obj = OBJ / ("core_" + src.stem + ".o")
        if force or _stale(obj, [src] + hdrs):
            _run([cxx, *CXX_FLAGS, *inc, "-c", str(src), "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    # Export the module init function only and bind the module's own references locally. The C++ standard library
    # templates instantiated in this module would otherwise be visible process-wide and get mixed with the copies
    # inside other extension modules (PyTorch), which crashes whichever module is imported second.
    vers = OBJ / "ovcore.map"
    vers.write_text("{ global: PyInit__ovcore; local: *; };\n")
    _run([cxx, "-shared", "-o", str(target), *map(str, objs), "-pthread", "-Wl,--version-script=%s" % vers, "-Wl,-Bsymbolic"])
    return target


def build_capi(force: bool = False) -> Path | None:
    """Link the native core (without the Python bindings) and the C API into ``lib/libopenvino_b200_c.so``."""
    capi = sorted((CSRC / "capi").glob("*.cpp"))
    if not capi:
        return None
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    target = LIB / "libopenvino_b200_c.so"
    core = [s for s in core_sources() if s.stem != "bind"]
    hdrs = sorted((CSRC / "core").glob("*.hpp")) + sorted((PKG / "include").rglob("*.h"))
    if not force and not _stale(target, capi + core + hdrs):
        return target
    cxx = os.environ.get("CXX", "g++")
    inc = ["-I", str(CSRC / "core")]

    def compile_one(src: Path) -> Path:
        obj = OBJ / ("capi_" + src.stem + ".o")
        if force or _stale(obj, [src] + hdrs):
            _run([cxx, *CXX_FLAGS, *inc, "-c", str(src), "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, capi + core))
    vers = OBJ / "ovcapi.map"
    vers.write_text("{ global: ov_*; local: *; };\n")
    _run([cxx, "-shared", "-o", str(target), *map(str, objs), "-pthread", "-Wl,--version-script=%s" % vers, "-Wl,-Bsymbolic"])
    return target


SANITIZERS = {"address": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "undefined": ["-fsanitize=undefined", "-fno-sanitize-recover=undefined"],
              "thread": ["-fsanitize=thread"]}


def build_native_test(test_source: Path, sanitize: str = "", force: bool = False, core_subset=None) -> Path:
    """Compile the native core and the C API together with one C++ test driver into a stand-alone executable, optionally
    under a sanitizer (``address`` = ASan + UBSan, ``undefined``, ``thread``; the reference's switch for the same is
    cmake/developer_package/compile_flags/sanitizer.cmake). Objects go to ``build/native_<sanitize>/``; nothing of the
    regular build is touched. ``core_subset`` names the core translation units to link (default: all of them plus the C API).
    ``python -m openvino_b200.build --sanitize=address tests/native/core_smoke.cpp`` does the same
    from the command line."""
    if sanitize and sanitize not in SANITIZERS:
        raise ValueError("unknown sanitizer %r (choose from %s)" % (sanitize, ", ".join(SANITIZERS)))
    test_source = Path(test_source).resolve()
    out_dir = OBJ / ("native_" + (sanitize or "plain"))
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = out_dir / (test_source.stem + ("" if core_subset is None else "." + "-".join(sorted(core_subset) or ["alone"])))
    core = [s for s in core_sources() if s.stem != "bind"]
    capi = sorted((CSRC / "capi").glob("*.cpp"))
    if core_subset is not None:           # a driver that needs only some translation units (and no C API)
        core, capi = [s for s in core if s.stem in set(core_subset)], []
    hdrs = sorted((CSRC / "core").glob("*.hpp")) + sorted((PKG / "include").rglob("*.h")) + sorted((CSRC / "cuda").glob("comm_layout.h"))
    if not force and not _stale(exe, core + capi + hdrs + [test_source]):
        return exe
    # the distribution's compiler knows where its sanitizer runtimes are; a compiler wrapper named by CXX may not
    cxx = os.environ.get("OVB_NATIVE_TEST_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else os.environ.get("CXX", "g++"))
    flags = ["-O1", "-g", "-std=c++17", "-fno-omit-frame-pointer", "-pthread", "-Wall", "-Wno-unused-function", *SANITIZERS.get(sanitize, [])]
    inc = ["-I", str(CSRC / "core"), "-I", str(PKG / "include"), "-I", str(CSRC / "cuda")]

    def compile_one(src: Path) -> Path:
        obj = out_dir / (src.parent.name + "_" + src.stem + ".o")
        if force or _stale(obj, [src] + hdrs):
            _run([cxx, *flags, *inc, "-c", str(src), "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, core + capi + [test_source]))
    _run([cxx, *flags, "-o", str(exe), *map(str, objs)])
    return exe


def kernel_resources(stem: str) -> dict:
    """Per-kernel resource usage parsed from the ptxas report of ``csrc/cuda/<stem>.cu``:
    ``{mangled name: {"registers", "stack", "spill_stores", "spill_loads", "static_smem"}}`` (empty when no report exists)."""
    import re
    path = OBJ / (stem + ".ptxas.txt")
    if not path.exists():
        return {}
    out = {}
    pat = re.compile(r"Compiling entry function '(\S+)' for 'sm_100a'.*?(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads"
                     r".*?Used (\d+) registers", re.S)
    text = path.read_text()
    for m in pat.finditer(text):
        line_end = text.find("\n", m.end())
        used = text[m.end():line_end if line_end >= 0 else len(text)]
        smem = re.search(r"(\d+) bytes smem", used)
        out[m.group(1)] = {"stack": int(m.group(2)), "spill_stores": int(m.group(3)), "spill_loads": int(m.group(4)), "registers": int(m.group(5)),
                           "static_smem": int(smem.group(1)) if smem else 0}
    return out


def build_selective(stats_csv, out_dir, stems=None, link: bool = True) -> Path:
    """Conditional compilation, the selective build: compile the kernel library with only the variants that an analysing
    run recorded (``utils/cc.py`` writes the statistics; lines ``gemm,<token tile>,<weight format>,<fp16>``). The library
    goes to ``out_dir/libovb_cuda.so`` (load it with ``OVB_CUDA_LIB``); variants that were left out are never instantiated.
    Role in the reference: the SELECTIVE_BUILD=ON stage driven by the collected statistics
    (src/common/conditional_compilation, cmake/developer_package/features.cmake)."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    keep = set()
    for line in Path(stats_csv).read_text().splitlines():
        parts = [p.strip() for p in line.split(",")]
        if len(parts) >= 4 and parts[0] == "gemm":
            keep.add((int(parts[1]), int(parts[2]), int(parts[3])))
    cond = " || ".join("(bt == %d && wmode == %d && f16 == %s)" % (bt, wm, "true" if f else "false") for bt, wm, f in sorted(keep)) or "false"
    (out_dir / "cc_selected.h").write_text(
        "// generated from %s: the GEMM variants of this selective build\n"
        "constexpr bool cc_gemm_selected(int bt, int wmode, bool f16) { return %s; }\n" % (Path(stats_csv).name, cond))
    nvcc = _nvcc()
    objs = []

    def compile_one(src: Path) -> Path:
        obj = out_dir / (src.stem + ".o")
        cmd = [nvcc, "-Xptxas", "-v", *NVCC_FLAGS, "-DOVB_CC_SELECTIVE", "-I", str(out_dir), "-I", str(CSRC / "cuda"), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout[-4000:], r.stderr[-8000:]))
        (out_dir / (src.stem + ".ptxas.txt")).write_text(r.stderr)
        return obj

    srcs = [s_ for s_ in cuda_sources() if stems is None or s_.stem in stems]
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    if not link:
        return out_dir
    vers = out_dir / "ovb_cuda.map"
    vers.write_text("{ global: ovb_*; local: *; };\n")
    target = out_dir / "libovb_cuda.so"
    _run([nvcc, "-shared", "-o", str(target), *map(str, objs), "-cudart", "static", "-Xlinker", "--version-script=%s" % vers])
    return target


def build_all(force: bool = False) -> None:
    build_cuda(force)
    build_core(force)
    build_capi(force)


if __name__ == "__main__":
    cc = [a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--cc-stats=")]
    if cc:
        out = ([a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--cc-out=")] or [str(PKG / "lib_selective")])[0]
        print("built:", build_selective(cc[0], out))
        sys.exit(0)
    if "--debug-bounds" in sys.argv:
        print("built:", build_cuda_debug(force="--force" in sys.argv))
        sys.exit(0)
    san = [a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--sanitize=")]
    if san:
        for src in [a for a in sys.argv[1:] if a.endswith(".cpp")]:
            print("built:", build_native_test(Path(src), san[0], force="--force" in sys.argv))
        sys.exit(0)
    build_all(force="--force" in sys.argv)
    print("built:", [p.name for p in LIB.glob("*.so")] + [p.name for p in PKG.glob("_ovcore*.so")])
