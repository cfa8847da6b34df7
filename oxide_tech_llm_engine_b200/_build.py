"""In-tree build and loading of the native extensions.

Two extensions live beside this file after a build:

* ``oxb_cuda``  - the sm_100a kernels (``csrc/kernels/*.cu`` + ``csrc/bindings.cpp``), compiled with
  ``-gencode arch=compute_100a,code=sm_100a``; nvcc cross-compiles them on a machine without a GPU.
* ``oxb_host``  - the C++ host runtime (block manager, radix prefix cache, scheduler core, GGUF
  block codecs); no CUDA dependency, so CPU-only tests can import it.

The shared objects are written to ``<package>/_ext/`` and are loaded from there; a content hash
of the sources is stored next to each one so that a stale object is rebuilt when a compiler is
available and reported loudly when it is not.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_ROOT = _PKG.parent
_CSRC = _ROOT / "csrc"
_EXT = _PKG / "_ext"

_lock = threading.Lock()
_loaded: dict[str, object] = {}

CUDA_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas",
    "-v",
]


def _sources(name: str) -> list[Path]:
    if name == "oxb_cuda":
        return sorted((_CSRC / "kernels").glob("*.cu")) + [_CSRC / "bindings.cpp"]
    if name == "oxb_host":
        return sorted((_CSRC / "host").glob("*.cpp"))
    raise KeyError(name)


def _headers(name: str) -> list[Path]:
    """Headers that the extension's sources include (a change in the other extension's headers must
    not make this one stale)."""
    if name == "oxb_host":
        return sorted((_CSRC / "host").glob("*.h"))
    return sorted(list((_CSRC / "common").glob("*")) + list((_CSRC / "kernels").glob("*.cuh")))


def source_hash(name: str) -> str:
    h = hashlib.sha256()
    for p in _sources(name) + _headers(name):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _so_path(name: str) -> Path:
    return _EXT / f"{name}.so"


def _stamp_path(name: str) -> Path:
    return _EXT / f"{name}.hash"


def is_fresh(name: str) -> bool:
    so, st = _so_path(name), _stamp_path(name)
    return so.exists() and st.exists() and st.read_text().strip() == source_hash(name)


def build(name: str, verbose: bool = False) -> Path:
    """Compile one extension in-tree (incremental through ninja)."""
    from torch.utils import cpp_extension

    _EXT.mkdir(exist_ok=True)
    build_dir = _EXT / f"build_{name}"
    build_dir.mkdir(exist_ok=True)
    srcs = [str(p) for p in _sources(name)]
    kwargs = dict(
        name=name,
        sources=srcs,
        extra_cflags=["-O3", "-std=c++17"],
        extra_include_paths=[str(_CSRC)],
        build_directory=str(build_dir),
        verbose=verbose,
        is_python_module=True,
    )
    if name == "oxb_cuda":
        kwargs["extra_cuda_cflags"] = CUDA_FLAGS
        kwargs["with_cuda"] = True
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 8))
    mod = cpp_extension.load(**kwargs)
    built = build_dir / f"{name}.so"
    if not built.exists():
        raise RuntimeError(f"build of {name} produced no {built}")
    so = _so_path(name)
    tmp = so.with_suffix(f".so.tmp{os.getpid()}")
    tmp.write_bytes(built.read_bytes())
    os.replace(tmp, so)
    _stamp_path(name).write_text(source_hash(name))
    _loaded[name] = mod
    return so


def _import_so(name: str):
    import torch  # noqa: F401  (libtorch symbols must be loaded first)

    spec = importlib.util.spec_from_file_location(name, _so_path(name))
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot load {_so_path(name)}")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules.setdefault(name, mod)
    return mod


class _BuildLock:
    """Lock between the processes of one job (one rank per GPU imports the package at the same time):
    only one of them rebuilds a stale extension, the others wait and then find it fresh."""

    def __enter__(self):
        import fcntl

        _EXT.mkdir(exist_ok=True)
        self.f = open(_EXT / ".build.lock", "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl

        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()
        return False


def load(name: str):
    """Return the extension module, building it first if it is missing or stale."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
        if not is_fresh(name):
            with _BuildLock():
                return _load_locked(name)
        return _load_locked(name)


def _load_locked(name: str):
    if not is_fresh(name):
        import shutil

        have_compiler = shutil.which("g++") is not None and (
            name != "oxb_cuda" or shutil.which("nvcc") is not None
        )
        if have_compiler and os.environ.get("OXB_NO_BUILD", "0") != "1":
            build(name)
            if name in _loaded:
                return _loaded[name]
        elif not _so_path(name).exists():
            raise ImportError(
                f"native extension {name} is not built and no compiler is available; "
                "run `python -c 'import __graft_entry__ as g; g.build()'` in the repo root"
            )
    mod = _import_so(name)
    _loaded[name] = mod
    return mod


def _noalloc_sources() -> list[Path]:
    return [_CSRC / "noalloc" / "paged_decode_noalloc.cu", _CSRC / "kernels" / "attn_decode.cu"]


def noalloc_hash() -> str:
    h = hashlib.sha256()
    for p in _noalloc_sources() + [_CSRC / "noalloc" / "oxb_noalloc.h", _CSRC / "kernels" / "attn.cuh"]:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def build_noalloc() -> Path:
    """Plain C-ABI shared library (no torch, no Python): `liboxb_noalloc.so`."""
    import subprocess

    _EXT.mkdir(exist_ok=True)
    so = _EXT / "liboxb_noalloc.so"
    cmd = ["nvcc", "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a",
           "-lineinfo", "-O3", "-std=c++17", "-cudart", "shared", "-o", str(so)]
    cmd += [str(p) for p in _noalloc_sources()]
    subprocess.run(cmd, check=True, capture_output=True)
    (_EXT / "liboxb_noalloc.hash").write_text(noalloc_hash())
    return so


def noalloc_lib_path() -> Path:
    """Path of the allocation-free C library, built on demand when a compiler is present."""
    import shutil

    so = _EXT / "liboxb_noalloc.so"
    st = _EXT / "liboxb_noalloc.hash"
    fresh = so.exists() and st.exists() and st.read_text().strip() == noalloc_hash()
    if not fresh:
        if shutil.which("nvcc") is not None and os.environ.get("OXB_NO_BUILD", "0") != "1":
            build_noalloc()
        elif not so.exists():
            raise ImportError("liboxb_noalloc.so is not built and nvcc is not available")
    return so


def cuda_ext():
    return load("oxb_cuda")


def host_ext():
    return load("oxb_host")
