"""Builds the CUDA kernels into shared libraries, in the tree, each on its first use.

Every ``*.cu`` under ``csrc/`` is compiled with nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``).  The files that the others lean on (the launch
attribute switch and the status word of bounded waits) form ``libshiso_base.so``; every other
file becomes a library of its own, ``libshiso_<file>.so``, linked against the base and built
the first time one of its entry points is called.  A model therefore compiles the kernels it
runs and no others: a design without recurrences never waits for the recurrence kernels.
The sources include no PyTorch headers: they export plain C launchers that take device
pointers and a stream, which Python calls through ctypes.  A hash of a file's source, the
headers and the flags is stored beside its object and its library; what does not match is rebuilt.
The build directory is ``csrc/_build`` when that is writable, else a per-user folder
under the system's temporary directory, so a read-only checkout or another user still
works.  A line is printed when compilation starts, per file, and at the end.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
BASE = "base"
BASE_SOURCES = ("elementwise.cu", "gemm_tcgen05.cu")  # define what every other file calls across files
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[shiso_llm_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("SHISO_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $SHISO_NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels cannot be built")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    override = os.environ.get("SHISO_BUILD_DIR")
    if override:
        if not _writable_dir(override):
            raise BuildError(f"SHISO_BUILD_DIR={override} is not writable")
        return override
    in_tree = os.path.join(CSRC, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"shiso_llm_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"neither {in_tree} nor {fallback} is writable: nowhere to build the CUDA kernels")


def module_of(source: str) -> str:
    """The library a source file goes into: the base, or one named after the file."""
    name = os.path.basename(source)
    return BASE if name in BASE_SOURCES else name[:-3]


def modules() -> list[str]:
    """Every library, the base first."""
    return [BASE] + sorted({module_of(s) for s in sources()} - {BASE})


def _module_sources(module: str) -> list[str]:
    if module == BASE:
        return [os.path.join(CSRC, f) for f in BASE_SOURCES]
    path = os.path.join(CSRC, module + ".cu")
    if not os.path.isfile(path):
        raise BuildError(f"no kernel file {module}.cu under {CSRC}")
    return [path]


def lib_name(module: str) -> str:
    return f"libshiso_{module}.so"


def _module_hash(module: str) -> str:
    h = hashlib.sha256()
    h.update(LINK_RULE.encode())
    for src in _module_sources(module):
        h.update(_object_hash(src).encode())
    if module != BASE:
        h.update(_module_hash(BASE).encode())
    return h.hexdigest()[:20]


def _fresh(directory: str, module: str) -> str | None:
    lib, stamp = os.path.join(directory, lib_name(module)), os.path.join(directory, lib_name(module) + ".hash")
    if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == _module_hash(module):
        return lib
    return None


def library_path(module: str = BASE, create: bool = True) -> str:
    """Path of an up-to-date library of one module, building it (and the base) first if needed."""
    # An up-to-date library in the tree wins even when the tree is read-only.
    found = _fresh(os.path.join(CSRC, "_build"), module)
    if found:
        return found
    d = build_dir()
    found = _fresh(d, module)
    if found:
        return found
    if not create:
        raise BuildError(f"the CUDA kernel library of {module} is not built")
    return build([module], d)[module]


def _object_hash(src: str) -> str:
    """What an object file depends on: its source, every header, the flags."""
    h = hashlib.sha256()
    for path in [src] + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:20]


LINK_RULE = "2"  # part of every library's hash: raised when the link line changes


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool) -> str:
    """Compiles one file, unless the object beside its stamp was built from the same source,
    headers and flags (a change to one kernel file then rebuilds that file only)."""
    stamp, want = obj + ".hash", _object_hash(src)
    if not verbose and os.path.isfile(obj) and os.path.isfile(stamp) and open(stamp).read().strip() == want:
        return ""
    cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{proc.stdout}\n{proc.stderr}")
    with open(stamp, "w") as f:
        f.write(want + "\n")
    return proc.stderr


def _link(nvcc: str, directory: str, module: str, base_lib: str | None) -> str:
    objs = [os.path.join(directory, os.path.basename(s)[:-3] + ".o") for s in _module_sources(module)]
    name = lib_name(module)
    tmp_lib = os.path.join(directory, f".{name}.{os.getpid()}")
    link = [nvcc, "-shared", "-o", tmp_lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xlinker", f"-soname={name}", "-Xlinker", "-rpath=$ORIGIN", "-Xlinker", "-Bsymbolic"]
    if base_lib is not None:
        # recorded by its soname; the loader has it in the process before any other library.  -Bsymbolic:
        # a library's calls to functions it defines itself (inline functions with static state
        # among them) stay inside it whatever else the process has loaded.
        link.append(base_lib)
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"linking {name} failed:\n{proc.stdout}\n{proc.stderr}")
    lib = os.path.join(directory, name)
    os.replace(tmp_lib, lib)
    with open(lib + ".hash", "w") as f:
        f.write(_module_hash(module) + "\n")
    return lib


def build(wanted: list[str] | None = None, directory: str | None = None, verbose: bool = False) -> dict:
    """Builds the libraries of ``wanted`` modules (None: all of them) and the base; returns
    module -> path."""
    nvcc = find_nvcc()
    d = directory or build_dir()
    wanted = modules() if wanted is None else list(dict.fromkeys([BASE] + list(wanted)))
    out, todo = {}, []
    for module in wanted:
        found = None if verbose else (_fresh(os.path.join(CSRC, "_build"), module) or _fresh(d, module))
        if found:
            out[module] = found
        else:
            todo.append(module)
    if not todo:
        return out
    srcs = [s for module in todo for s in _module_sources(module)]
    started = time.time()
    _say(f"compiling {len(srcs)} CUDA file(s) for sm_100a into {d}: {', '.join(os.path.basename(s) for s in srcs)} (first use)")
    objs = [os.path.join(d, os.path.basename(s)[:-3] + ".o") for s in srcs]
    log = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(os.cpu_count() or 4, 16, len(srcs))) as pool:
        futures = {pool.submit(_compile_one, nvcc, s, o, verbose): s for s, o in zip(srcs, objs)}
        for fut in concurrent.futures.as_completed(futures):
            log.append(fut.result())
            _say(f"  compiled {os.path.basename(futures[fut])} ({time.time() - started:.0f} s)")
    if BASE in todo:
        out[BASE] = _link(nvcc, d, BASE, None)
    for module in todo:
        if module != BASE:
            out[module] = _link(nvcc, d, module, out[BASE])
    if verbose:
        with open(os.path.join(d, "ptxas.log"), "a") as f:
            f.write("\n".join(log))
    _say(f"built {', '.join(lib_name(m) for m in todo)} in {time.time() - started:.0f} s")
    return out


_EXPORT = None


def exports() -> dict:
    """Entry point -> module, read off the sources (every launcher is marked ``SHISO_API``)."""
    global _EXPORT
    if _EXPORT is None:
        import re

        pattern = re.compile(r"SHISO_API\s+[\w\s\*]*?\b(shiso_\w+)\s*\(")
        found = {}
        for src in sources():
            with open(src, "r", encoding="utf-8") as f:
                for name in pattern.findall(f.read()):
                    found[name] = module_of(src)
        _EXPORT = found
    return _EXPORT
