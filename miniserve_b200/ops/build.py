"""Compiles the native libraries of this package on demand, in-tree.

Each *module* is one shared library made from a few source files under ``csrc/``:

- ``host``: the C++ block allocator, block tables and step packer (g++ only, no CUDA);
- ``kernels``: the CUDA kernels every model needs, for sm_100a;
- further modules are compiled only when a model needs them (for instance the bfloat16
  attention kernels for one head size), so a first call compiles what that model uses.

A library is rebuilt when the hash of its sources and flags changes. Objects are compiled
in parallel and a line is printed per file, because a first build takes a while. The
libraries are written under ``miniserve_b200/_native/``; if that folder cannot be written,
under a per-user folder in the temporary directory.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
_IN_TREE = Path(__file__).resolve().parent.parent / "_native"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra"]


@dataclass(frozen=True)
class Module:
    name: str
    sources: tuple[str, ...]
    defines: tuple[str, ...] = ()
    cuda: bool = True
    extra_deps: tuple[str, ...] = field(default=("common.cuh",))


HOST = Module("host", ("host_core.cpp",), cuda=False, extra_deps=())
KERNELS = Module(
    "kernels",
    ("runtime.cu", "elementwise.cu", "rope_kv.cu", "gemm_f32.cu", "gemm_skinny.cu", "attention_rowwise.cu",
     "sampling.cu"),
)


# head sizes whose attention kernels __graft_entry__.build() compiles ahead of time (the tests'
# and the benchmark's); any other multiple of 16 up to 256 is compiled when a model first needs it
PREBUILT_HEAD_DIMS = (16, 32, 48, 64, 80, 128, 256)


GEMM_TC = Module("gemm_tc", ("gemm_tc.cu",))
ATTN_TC = Module("attn_tc", ("attention_tc.cu",))


def all_modules() -> list[Module]:
    """Every module of the package (what ``__graft_entry__.build`` compiles)."""
    from .attention_bf16 import module_for

    return [HOST, KERNELS, GEMM_TC, ATTN_TC] + [module_for(d) for d in PREBUILT_HEAD_DIMS]


def log(msg: str) -> None:
    print(f"[miniserve_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("MINISERVE_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError(
        "nvcc was not found (looked at $MINISERVE_NVCC, PATH and $CUDA_HOME/bin); the CUDA kernels of "
        "miniserve_b200 cannot be built and there is no other implementation to fall back to")


def build_dir() -> Path:
    override = os.environ.get("MINISERVE_BUILD_DIR")
    cands = [Path(override)] if override else [_IN_TREE]
    cands.append(Path(tempfile.gettempdir()) / f"miniserve_b200-native-{os.getuid()}")
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".write-test-{os.getpid()}"
            probe.write_text("x")
            probe.unlink()
            return d
        except OSError:
            continue
    raise RuntimeError(f"no writable build folder among {cands}")


def _digest(mod: Module) -> str:
    h = hashlib.sha256()
    flags = NVCC_FLAGS if mod.cuda else CXX_FLAGS
    h.update(repr((flags, mod.defines, mod.sources)).encode())
    for name in mod.sources + mod.extra_deps:
        h.update((CSRC / name).read_bytes())
    # headers that a source includes beyond common.cuh
    for inc in sorted(CSRC.glob("*.cuh")):
        if inc.name not in mod.extra_deps:
            h.update(inc.read_bytes())
    return h.hexdigest()[:20]


def library_path(mod: Module) -> Path:
    return build_dir() / f"libms_{mod.name}.so"


def _run(cmd: list[str], what: str) -> None:
    t0 = time.time()
    log(f"compiling {what} ...")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"building {what} failed:\n$ {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    log(f"compiled {what} in {time.time() - t0:.1f} s")


def debug_checks() -> bool:
    """MINISERVE_DEBUG=1: the CUDA libraries are compiled with -DMS_DEBUG_CHECKS (bounds checks that raise
    the status word, see ``csrc/common.cuh``) under names of their own, beside the ordinary ones."""
    return os.environ.get("MINISERVE_DEBUG", "0") == "1"


def host_sanitizers() -> bool:
    """MINISERVE_HOST_SANITIZE=1: the host core is compiled with AddressSanitizer and
    UndefinedBehaviorSanitizer (the process that loads it must have the sanitizer's runtime preloaded)."""
    return os.environ.get("MINISERVE_HOST_SANITIZE", "0") == "1"


def _variant(mod: Module) -> tuple[Module, list[str]]:
    """The module as it is built under the debugging switches, and extra compiler flags."""
    if mod.cuda and debug_checks():
        return Module(mod.name + "_dbg", mod.sources, mod.defines + ("MS_DEBUG_CHECKS",), mod.cuda, mod.extra_deps), []
    if not mod.cuda and host_sanitizers():
        return (Module(mod.name + "_san", mod.sources, mod.defines, mod.cuda, mod.extra_deps),
                ["-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-g"])
    return mod, []


def ensure_built(mod: Module, verbose_ptxas: bool = False) -> Path:
    """Path of the module's shared library, compiling it first if it is missing or stale."""
    mod, extra_flags = _variant(mod)
    out_dir = build_dir()
    lib = out_dir / f"libms_{mod.name}.so"
    stamp = out_dir / f"libms_{mod.name}.stamp"
    digest = _digest(mod)
    if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest and not verbose_ptxas:
        return lib
    with open(out_dir / f".{mod.name}.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest and not verbose_ptxas:
            return lib  # another process built it while we waited
        obj_dir = out_dir / f"obj_{mod.name}"
        obj_dir.mkdir(exist_ok=True)
        defines = [f"-D{d}" for d in mod.defines]
        if mod.cuda:
            nvcc = find_nvcc()
            jobs = []
            for src in mod.sources:
                obj = obj_dir / (Path(src).stem + ".o")
                cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", str(CSRC), "-c", str(CSRC / src), "-o", str(obj)]
                if verbose_ptxas:
                    cmd[1:1] = ["-Xptxas", "-v"]
                jobs.append((cmd, f"{mod.name}/{src}", obj))
            with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
                list(pool.map(lambda j: _run(j[0], j[1]), jobs))
            tmp = lib.with_suffix(f".tmp{os.getpid()}.so")
            _run([nvcc, "-shared", "-o", str(tmp), *[str(j[2]) for j in jobs]], f"{mod.name} (link)")
        else:
            cxx = shutil.which("g++") or shutil.which("c++")
            if cxx is None:
                raise RuntimeError("no C++ compiler (g++) found; the host core of miniserve_b200 cannot be built")
            tmp = lib.with_suffix(f".tmp{os.getpid()}.so")
            _run([cxx, *CXX_FLAGS, *extra_flags, *defines, "-shared", "-o", str(tmp), *[str(CSRC / s) for s in mod.sources]],
                 f"{mod.name}")
        os.replace(tmp, lib)
        stamp.write_text(digest)
    return lib
