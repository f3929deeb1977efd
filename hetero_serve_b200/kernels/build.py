"""Builds the CUDA library of this package for sm_100a, in the tree, on first use.

Every ``.cu`` file under ``csrc/`` is compiled with ``nvcc -gencode
arch=compute_100a,code=sm_100a`` into one object, the objects are linked into
``csrc/_build/libhetero_serve_b200-<hash>.so`` and the library is opened with
``ctypes``.  The hash covers the sources and the flags, so a stale library is never
loaded.  Nothing is taken from the user's home directory: a fresh checkout owned by
any user builds in place (or under the system's temporary directory when the
checkout is read-only).  The sources include no framework headers, so a cold build
takes well under a minute; a line is printed per step so that a caller sees progress.

The reference compiles its kernels at first use as well, through
``torch.utils.cpp_extension.load_inline`` with no architecture flag
(heteroserve/model/paged_attn.py:202-241); this build names sm_100a and nothing else.
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
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]
if os.environ.get("HETERO_SERVE_PHASE_MARKS") == "1":      # a tuning build (see common.cuh)
    NVCC_FLAGS = NVCC_FLAGS + ["-DHS_PHASE_MARKS"]
    LIB_STEM = "libhetero_serve_b200_marks"                # kept beside the product library
else:
    LIB_STEM = "libhetero_serve_b200"


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[hetero_serve_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("HETERO_SERVE_NVCC"), shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    cuda_home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH")
    if cuda_home and (Path(cuda_home) / "bin" / "nvcc").is_file():
        return str(Path(cuda_home) / "bin" / "nvcc")
    raise BuildError("nvcc not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels of "
                     "hetero_serve_b200 cannot be built, and there is no fallback")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def source_hash() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> Path:
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"hetero_serve_b200-{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def library_path() -> Path:
    return _build_dir() / f"{LIB_STEM}-{source_hash()}.so"


def _run(cmd: list[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n$ {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def build(force: bool = False, verbose: bool = True) -> Path:
    """Compile (if needed) and return the path of the shared library."""
    lib = library_path()
    if lib.is_file() and not force:
        return lib
    nvcc = find_nvcc()
    srcs = sources()
    if not srcs:
        raise BuildError(f"no CUDA sources in {CSRC}")
    bdir = lib.parent
    tag = lib.stem.rsplit("-", 1)[-1]
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} ...")

    def compile_one(src: Path) -> Path:
        obj = bdir / f"{src.stem}-{tag}.o"
        _run([nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
             f"compiling {src.name}")
        if verbose:
            _say(f"  {src.name} done ({time.time() - t0:.0f}s)")
        return obj

    workers = min(len(srcs), max(1, (os.cpu_count() or 2)))
    with concurrent.futures.ThreadPoolExecutor(workers) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = bdir / f".{lib.name}.{os.getpid()}"
    _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs)], "linking")
    os.replace(tmp, lib)
    for o in objs:
        try:
            o.unlink()
        except OSError:
            pass
    # older libraries of other source versions are of no use to anyone, nor are the objects an
    # interrupted build left behind (an hour old: no build still running wrote them)
    stale = [old for old in bdir.glob(f"{LIB_STEM}-*.so") if old != lib]
    stale += [o for o in bdir.glob("*.o") if time.time() - o.stat().st_mtime > 3600]
    for old in stale:
        try:
            old.unlink()
        except OSError:
            pass
    if verbose:
        _say(f"built {lib.name} in {time.time() - t0:.0f}s")
    return lib


def build_extension(name: str, srcs: list[str | Path], verbose: bool = False) -> Path:
    """Compile CUDA sources that are not part of this package into a library of their own,
    with the package's flags for sm_100a and ``csrc/`` on the include path (``common.cuh``
    and ``tcgen05.cuh`` are there for them).  This is how a part defined elsewhere — another
    architecture's mixer, a test's toy part — brings its kernels: it builds them here and
    opens them with :meth:`CudaOps.load_extension`; nothing in this package changes.

    The library is named after a hash of its sources and kept in the build folder, so a
    second call returns at once."""
    nvcc = find_nvcc()
    paths = [Path(s) for s in srcs]
    h = hashlib.sha256()
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    for p in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    bdir = _build_dir()
    lib = bdir / f"lib{name}-{h.hexdigest()[:16]}.so"
    if lib.is_file():
        return lib
    if verbose:
        _say(f"compiling extension {name} ({len(paths)} files) for sm_100a ...")
    tmp = bdir / f".{lib.name}.{os.getpid()}"
    _run([nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-shared", "-o", str(tmp),
          *map(str, paths)], f"compiling extension {name}")
    os.replace(tmp, lib)
    return lib
