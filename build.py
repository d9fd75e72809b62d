#!/usr/bin/env python
"""In-tree build of the native core.

Generates a ninja file for every C++/CUDA source under ``csrc/`` and links

* ``pplx_garden/_native.<abi>.so``   the Python extension (pybind11),
* ``pplx_garden/libpplx_noalloc.so`` plain C entry points (when their source exists),
* ``bin/pplx-fabric-debug`` and ``bin/pplx-unigram-encode`` command line tools, and
  ``bin/pplx-core-tests``, the native unit tests
  (when their sources exist).

CUDA is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``); nvcc
cross-compiles, so the build works on machines without a GPU. The CUDA runtime is linked
statically and the driver API is resolved at run time, so the extension imports on
machines without a driver as well.

The reference builds the same pieces with cargo + a cc/nvcc build script
(p2p-all-to-all/a2a-kernels/build.rs:9-22, python-ext/Cargo.toml).

Usage: ``python build.py [--verbose] [--clean] [--jobs N]``
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _pybind_include() -> str:
    import pybind11

    return pybind11.get_include()


def _sources() -> dict[str, list[Path]]:
    groups: dict[str, list[Path]] = {"ext": [], "noalloc": [], "fabric_debug": [], "unigram_cli": [], "core_tests": []}
    for path in sorted(CSRC.rglob("*")):
        if path.suffix not in (".cpp", ".cu"):
            continue
        rel = path.relative_to(CSRC)
        if rel.parts[0] == "noalloc":
            groups["noalloc"].append(path)
        elif rel.parts[0] == "tools":
            if path.stem == "fabric_debug":
                groups["fabric_debug"].append(path)
            elif path.stem == "unigram_encode":
                groups["unigram_cli"].append(path)
            elif path.stem == "core_tests":
                groups["core_tests"].append(path)
        else:
            groups["ext"].append(path)
    return groups


def _has_header(name: str) -> bool:
    return any((Path(d) / name).exists() for d in ("/usr/include", "/usr/local/include"))


def _sanitizer_compiler(sanitize: str) -> str:
    """A g++ that can link -fsanitize=<sanitize> (the runtime library is not part of every install)."""
    import tempfile

    for cxx in dict.fromkeys([os.environ.get("CXX", "g++"), "/usr/bin/g++", "g++"]):
        with tempfile.TemporaryDirectory(dir=BUILD) as tmp:
            src = Path(tmp) / "probe.cpp"
            src.write_text("int main() { return 0; }\n")
            probe = subprocess.run([cxx, f"-fsanitize={sanitize}", str(src), "-o", str(Path(tmp) / "probe")],
                                   capture_output=True)
            if probe.returncode == 0:
                return cxx
    raise RuntimeError(f"no g++ here can link -fsanitize={sanitize}")


def write_ninja(verbose: bool, sanitize: str | None = None) -> Path:
    BUILD.mkdir(exist_ok=True)
    py_inc = sysconfig.get_paths()["include"]
    ext_suffix = sysconfig.get_config_var("EXT_SUFFIX")
    common_inc = ["-Icsrc", f"-I{CUDA_HOME}/include"]
    defines = []
    if _has_header("infiniband/verbs.h"):
        defines.append("-DPPLX_HAVE_VERBS=1")
    if _has_header("rdma/fabric.h"):
        defines.append("-DPPLX_HAVE_LIBFABRIC=1")
    cxxflags = ["-std=c++17", "-O3", "-g1", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread",
                "-fvisibility=hidden"] + defines
    nvflags = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC",
               "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
               "-Xptxas", "-v" if verbose else "-warn-spills"] + NVCC_ARCH + defines
    lines = [
        "ninja_required_version = 1.3",
        f"cxx = {os.environ.get('CXX', 'g++')}",
        f"nvcc = {CUDA_HOME}/bin/nvcc",
        f"cxxflags = {' '.join(cxxflags + common_inc)}",
        f"pyflags = -I{py_inc} -I{_pybind_include()}",
        f"nvflags = {' '.join(nvflags + common_inc)}",
        f"ldflags = -L{CUDA_HOME}/lib64 -lcudart_static -ldl -lrt -lpthread",
        "rule cxx",
        "  command = $cxx -MMD -MF $out.d $cxxflags $extra -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = CXX $in",
        "rule nvcc",
        "  command = $nvcc -MD -MF $out.d $nvflags -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = NVCC $in",
        "rule link_shared",
        "  command = $cxx -shared -o $out $in $ldflags -Wl,--exclude-libs,ALL",
        "  description = LINK $out",
        "rule link_exe",
        "  command = $cxx -o $out $in $ldflags",
        "  description = LINK $out",
        "",
    ]
    if sanitize:
        # The host code once more with a sanitizer (address, thread or undefined), for the native
        # unit tests only: kernels and CUDA runtime calls are not instrumented.
        san = ["-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={sanitize}", "-fPIC", "-Wall",
               "-Wno-unused-function", "-pthread"] + defines
        lines += [
            f"sancxx = {_sanitizer_compiler(sanitize)}",
            f"sanflags = {' '.join(san + common_inc)}",
            "rule cxx_san",
            "  command = $sancxx -MMD -MF $out.d $sanflags -c $in -o $out",
            "  depfile = $out.d",
            "  deps = gcc",
            "  description = CXX($sanitize) $in".replace("$sanitize", sanitize),
            "rule link_san",
            f"  command = $sancxx -fsanitize={sanitize} -o $out $in $ldflags",
            "  description = LINK $out",
            "",
        ]
    groups = _sources()

    def compile_group(paths: list[Path], tag: str) -> list[str]:
        objs = []
        for src in paths:
            rel = src.relative_to(CSRC)
            obj_abs = BUILD / tag / rel.with_suffix(rel.suffix + ".o")
            obj_abs.parent.mkdir(parents=True, exist_ok=True)
            # relative paths: the tree may be copied to another location with its build/
            obj = obj_abs.relative_to(ROOT)
            src = src.relative_to(ROOT)
            if src.suffix == ".cu":
                lines.append(f"build {obj}: nvcc {src}")
            else:
                lines.append(f"build {obj}: cxx {src}")
                if rel.parts[0] == "bindings":
                    lines.append("  extra = $pyflags")
            objs.append(str(obj))
        return objs

    targets = []
    ext_objs = compile_group(groups["ext"], "ext")
    ext_out = Path("pplx_garden") / f"_native{ext_suffix}"
    lines.append(f"build {ext_out}: link_shared {' '.join(ext_objs)}")
    targets.append(str(ext_out))

    # Object files shared with the command line tools (everything except the bindings).
    core_objs = [o for o in ext_objs if "/bindings/" not in o]

    if groups["noalloc"]:
        objs = compile_group(groups["noalloc"], "noalloc")
        out = Path("pplx_garden") / "libpplx_noalloc.so"
        lines.append(f"build {out}: link_shared {' '.join(objs)}")
        targets.append(str(out))
    for key, name in (("fabric_debug", "pplx-fabric-debug"), ("unigram_cli", "pplx-unigram-encode"),
                      ("core_tests", "pplx-core-tests")):
        if groups[key]:
            objs = compile_group(groups[key], key)
            out = Path("bin") / name
            (ROOT / "bin").mkdir(exist_ok=True)
            lines.append(f"build {out}: link_exe {' '.join(objs + core_objs)}")
            targets.append(str(out))
    if sanitize and groups["core_tests"]:
        san_objs = []
        for src in [p for p in groups["ext"] if "bindings" not in p.relative_to(CSRC).parts] + groups["core_tests"]:
            rel = src.relative_to(CSRC)
            if src.suffix == ".cu":
                # device code and its host stubs as built above
                san_objs.append(str((BUILD / "ext" / rel.with_suffix(rel.suffix + ".o")).relative_to(ROOT)))
                continue
            obj = (BUILD / f"san-{sanitize}" / rel.with_suffix(rel.suffix + ".o"))
            obj.parent.mkdir(parents=True, exist_ok=True)
            lines.append(f"build {obj.relative_to(ROOT)}: cxx_san {src.relative_to(ROOT)}")
            san_objs.append(str(obj.relative_to(ROOT)))
        out = Path("bin") / f"pplx-core-tests-{sanitize}"
        lines.append(f"build {out}: link_san {' '.join(san_objs)}")
        targets.append(str(out))
    lines.append(f"default {' '.join(targets)}")
    ninja = BUILD / "build.ninja"
    ninja.write_text("\n".join(lines) + "\n")
    return ninja


def build(verbose: bool = False, jobs: int | None = None, clean: bool = False, sanitize: str | None = None) -> None:
    if clean and BUILD.exists():
        shutil.rmtree(BUILD)
    ninja = write_ninja(verbose, sanitize)
    cmd = ["ninja", "-f", str(ninja)]
    if jobs:
        cmd += ["-j", str(jobs)]
    if verbose:
        cmd.append("-v")
    subprocess.run(cmd, check=True, cwd=ROOT)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--verbose", action="store_true", help="show commands and ptxas resource usage")
    ap.add_argument("--clean", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--sanitize", choices=["address", "thread", "undefined"], default=None,
                    help="also build bin/pplx-core-tests-<sanitizer>: the host code and its native unit tests "
                         "(engine threads, imm counters, sharding, ...) under that sanitizer")
    args = ap.parse_args()
    build(args.verbose, args.jobs, args.clean, args.sanitize)


if __name__ == "__main__":
    main()
