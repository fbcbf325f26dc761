"""Build the native parts in-tree.

* ``lorax_b200/_lx_kernels.so``  every CUDA kernel, compiled by nvcc for sm_100a only and exported through a
  plain C ABI (loaded with ctypes, no Python headers needed, seconds per file).
* ``lorax_b200/bin/lorax-router`` and ``lorax_b200/bin/lorax-launcher``, plus ``lorax_b200/_lx_host.so`` with
  the C++ scheduler / allocator / radix-trie exported for the Python bindings and tests.

Usage: ``python -m lorax_b200.csrc.build [--force] [--verbose] [--only kernels|host]``
"""

from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import json
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parent
KERNEL_DIR = HERE / "kernels"
HOST_DIR = HERE / "host"
BUILD_DIR = PKG / "build"
KERNELS_SO = PKG / "_lx_kernels.so"
HOST_SO = PKG / "_lx_host.so"
BIN_DIR = PKG / "bin"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _run(cmd, verbose: bool, log_path: Path | None = None, quiet: bool = False) -> str:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path is not None:
        log_path.write_text(proc.stdout)
    if proc.returncode != 0:
        if not quiet:
            sys.stderr.write(" ".join(map(str, cmd)) + "\n" + proc.stdout + "\n")
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")
    if verbose:
        print(proc.stdout)
    return proc.stdout


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(KERNEL_DIR.glob("*.cu"))
    headers = sorted(KERNEL_DIR.glob("*.cuh")) + sorted(KERNEL_DIR.glob("*.h"))
    BUILD_DIR.mkdir(exist_ok=True)
    stamp = BUILD_DIR / "kernels.sha256"
    digest = _digest(sources + headers + [Path(__file__)])
    if not force and KERNELS_SO.exists() and stamp.exists() and stamp.read_text() == digest:
        return KERNELS_SO
    nvcc = _nvcc()
    hdr_digest = _digest(headers)

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / (src.stem + ".o")
        ostamp = BUILD_DIR / (src.stem + ".sha256")
        d = _digest([src]) + hdr_digest
        if not force and obj.exists() and ostamp.exists() and ostamp.read_text() == d:
            return obj
        _run([nvcc, *NVCC_FLAGS, "-I", str(KERNEL_DIR), "-c", str(src), "-o", str(obj)], verbose,
             BUILD_DIR / (src.stem + ".ptxas.log"))
        ostamp.write_text(d)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as ex:
        objs = list(ex.map(compile_one, sources))
    _run([nvcc, "-shared", "-o", str(KERNELS_SO), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
          "-Xcompiler", "-fPIC", "-lcudart_static", "-ldl", "-lrt", "-lpthread"], verbose)
    stamp.write_text(digest)
    return KERNELS_SO


def _unicode_tables():
    """`unicode_tables.hpp` (character classes, case and normalisation tables of the router's tokenizer) is generated from Python's
    `unicodedata` when it is missing or older than its generator."""
    out, gen = HOST_DIR / "unicode_tables.hpp", HOST_DIR / "gen_unicode_tables.py"
    if out.exists() and out.stat().st_mtime >= gen.stat().st_mtime:
        return
    import importlib.util
    spec = importlib.util.spec_from_file_location("gen_unicode_tables", gen)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.main(str(out))


def build_host(force: bool = False, verbose: bool = False):
    sources = sorted(HOST_DIR.glob("*.cpp"))
    if not sources:
        return None
    # the protobuf codec of the wire contract is generated from proto/generate.proto
    from lorax_b200.server import protogen
    protogen.main([str(HOST_DIR / "pb_gen.hpp")])
    _unicode_tables()
    # the OpenAPI document the router serves at /docs and /api-doc/openapi.json is the one of the documentation
    spec = PKG.parent / "docs" / "reference" / "openapi.json"
    body = json.dumps(json.loads(spec.read_text()), separators=(",", ":")) if spec.exists() else '{"openapi":"3.0.3","info":{"title":"lorax-b200","version":"0.2.0"},"paths":{}}'
    chunks = [body[i:i + 8000] for i in range(0, len(body), 8000)]       # string literals are limited in length by the standard
    gen = "// generated from docs/reference/openapi.json by csrc/build.py\n#pragma once\nstatic const char* const kOpenApiChunks[] = {\n" + \
        "".join('  R"OAPI(' + c + ')OAPI",\n' for c in chunks) + "  nullptr};\n"
    out = HOST_DIR / "openapi_gen.hpp"
    if not out.exists() or out.read_text() != gen:
        out.write_text(gen)
    headers = sorted(HOST_DIR.glob("*.h")) + sorted(HOST_DIR.glob("*.hpp"))
    BUILD_DIR.mkdir(exist_ok=True)
    BIN_DIR.mkdir(exist_ok=True)
    stamp = BUILD_DIR / "host.sha256"
    digest = _digest(sources + headers + [Path(__file__)])
    outs = [HOST_SO, BIN_DIR / "lorax-router", BIN_DIR / "lorax-launcher"]
    if not force and all(o.exists() for o in outs) and stamp.exists() and stamp.read_text() == digest:
        return HOST_SO
    cxx = os.environ.get("CXX", "g++")
    mains = {"router_main.cpp": "lorax-router", "launcher_main.cpp": "lorax-launcher"}
    lib_srcs = [s for s in sources if s.name not in mains]

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / ("host_" + src.stem + ".o")
        _run([cxx, *CXX_FLAGS, "-I", str(HOST_DIR), "-c", str(src), "-o", str(obj)], verbose)
        return obj

    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        objs = dict(zip([s.name for s in sources], ex.map(compile_one, sources)))
    lib_objs = [str(objs[s.name]) for s in lib_srcs]
    # -Bsymbolic: the library is loaded into Python processes next to other C++ libraries (torch); its own
    # definitions must win over same-named vague-linkage symbols already in the process.
    _run([cxx, "-shared", "-o", str(HOST_SO), *lib_objs, "-pthread", "-Wl,-Bsymbolic"], verbose)
    for main_src, exe in mains.items():
        if main_src in objs:
            _run([cxx, "-o", str(BIN_DIR / exe), str(objs[main_src]), *lib_objs, "-pthread"], verbose)
    stamp.write_text(digest)
    return HOST_SO


class SanitizerUnavailable(RuntimeError):
    pass


def build_host_selftest(sanitizer: str, verbose: bool = False) -> Path:
    """The host code's self test (`csrc/host/selftest/selftest_main.cpp` + the C API) under a sanitizer: "address" (with
    undefined-behaviour checks) or "thread".  Returns the binary; running it prints OK and exits 0 when nothing was found."""
    from lorax_b200.server import protogen
    protogen.main([str(HOST_DIR / "pb_gen.hpp")])
    _unicode_tables()
    # the OpenAPI document the router serves at /docs and /api-doc/openapi.json is the one of the documentation
    spec = PKG.parent / "docs" / "reference" / "openapi.json"
    body = json.dumps(json.loads(spec.read_text()), separators=(",", ":")) if spec.exists() else '{"openapi":"3.0.3","info":{"title":"lorax-b200","version":"0.2.0"},"paths":{}}'
    chunks = [body[i:i + 8000] for i in range(0, len(body), 8000)]       # string literals are limited in length by the standard
    gen = "// generated from docs/reference/openapi.json by csrc/build.py\n#pragma once\nstatic const char* const kOpenApiChunks[] = {\n" + \
        "".join('  R"OAPI(' + c + ')OAPI",\n' for c in chunks) + "  nullptr};\n"
    out = HOST_DIR / "openapi_gen.hpp"
    if not out.exists() or out.read_text() != gen:
        out.write_text(gen)
    BUILD_DIR.mkdir(exist_ok=True)
    flags = {"address": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "thread": ["-fsanitize=thread"]}[sanitizer]
    out = BUILD_DIR / f"host_selftest_{sanitizer}"
    srcs = [HOST_DIR / "selftest" / "selftest_main.cpp", HOST_DIR / "capi.cpp"]
    stamp = BUILD_DIR / f"host_selftest_{sanitizer}.sha256"
    digest = _digest(srcs + sorted(HOST_DIR.glob("*.hpp")) + [Path(__file__)])
    if out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    # not every toolchain ships the sanitizer runtimes: take the first compiler that links against them
    last = None
    for cxx in dict.fromkeys([os.environ.get("CXX", "g++"), "g++", "/usr/bin/g++", "clang++"]):
        if shutil.which(cxx) is None:
            continue
        try:
            _run([cxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, "-I", str(HOST_DIR), *map(str, srcs), "-o", str(out),
                  "-pthread"], verbose, quiet=True)
            stamp.write_text(digest)
            return out
        except RuntimeError as e:
            last = e
    raise SanitizerUnavailable(f"no compiler on this machine links -fsanitize={sanitizer}: {last}")


def build_all(force: bool = False, verbose: bool = False):
    k = build_kernels(force, verbose)
    h = build_host(force, verbose)
    return k, h


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--only", choices=["kernels", "host"])
    a = ap.parse_args(argv)
    if a.only != "host":
        print(build_kernels(a.force, a.verbose))
    if a.only != "kernels":
        print(build_host(a.force, a.verbose))


if __name__ == "__main__":
    main()
