"""Compiles the engine's CUDA sources for sm_100a with nvcc and loads them.

Each `.cu` file becomes one shared library, built the first time an operation
from it is used and kept beside the sources under `csrc/_build/` (or, when that
folder cannot be written, under the system's temporary folder).  The file name
carries a hash of the source, of the headers beside it (*.cuh, *.h) and of the flags, so an
edited source is rebuilt and a stale library is never loaded.  There is no
fallback: when a library can be neither found nor built, loading raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-lineinfo", "-std=c++17", "--shared", "-Xcompiler", "-fPIC"]
SOURCES = ("embed_norm", "rope_cache", "attention", "activation", "gemm_f32", "gemm_bf16", "gemm_tc5", "gemm_tc5_pair", "sampling",
           "memprobe")
# sources compiled once per value of a constant; the values here are what build_all() prepares,
# any other allowed value is compiled when a model first needs it
VARIANTS = {"flash_attn": [{"FA_HD": 128}, {"FA_HD": 64}, {"FA_HD": 32}, {"FA_HD": 16}],
            "flash_tc5": [{"FA_HD": 128}, {"FA_HD": 64}],
            "flash_decode_tma": [{"FA_HD": 128}, {"FA_HD": 64}]}
EXTRA_LIBS = {}

_loaded = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg):
    print(f"[vllm-lite_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
                     "the engine has no path without its CUDA libraries")


def _variant(defines) -> str:
    """Part of a library's file name that tells its compile-time constants, e.g. 'FA_HD128'."""
    return "_".join(f"{k}{v}" for k, v in sorted((defines or {}).items()))


def _digest(name: str, defines=None) -> str:
    h = hashlib.sha256()
    h.update((CSRC / f"{name}.cu").read_bytes())
    for header in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(header.read_bytes())
    h.update(" ".join(NVCC_FLAGS + EXTRA_LIBS.get(name, [])).encode())
    h.update(_variant(defines).encode())
    return h.hexdigest()[:12]


def _build_dirs():
    yield CSRC / "_build"
    yield Path(tempfile.gettempdir()) / f"vllm_lite_b200_build_{os.getuid()}"


def library_path(name: str, defines=None) -> Path:
    """Path of the up-to-date library of `name` (compiled with -D<key>=<value> for `defines`),
    building it if it is absent."""
    if not (CSRC / f"{name}.cu").is_file():
        raise BuildError(f"no CUDA source {name}.cu under {CSRC}")
    stem = name + ("." + _variant(defines) if defines else "")
    fname = f"{stem}.{_digest(name, defines)}.so"
    for d in _build_dirs():
        if (d / fname).is_file():
            return d / fname
    last = None
    for d in _build_dirs():
        try:
            d.mkdir(parents=True, exist_ok=True)
            if not os.access(d, os.W_OK):
                continue
            return _compile(name, d / fname, stem, defines)
        except (OSError, BuildError) as e:   # try the next folder; report the last failure
            last = e
            if isinstance(e, BuildError) and "nvcc" in str(e) and "not found" in str(e):
                break
    raise BuildError(f"could not build {name}.cu: {last}")


def _compile(name: str, out: Path, stem: str, defines=None) -> Path:
    nvcc = find_nvcc()
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    dflags = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    cmd = ([nvcc] + NVCC_FLAGS + dflags + ["-I", str(CSRC), "-o", str(tmp), str(CSRC / f"{name}.cu")]
           + EXTRA_LIBS.get(name, []))
    _say(f"compiling {name}.cu {' '.join(dflags)} for sm_100a ...".replace("  ", " "))
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env={**os.environ, "TMPDIR": tempfile.gettempdir()})
    while True:
        try:
            log, _ = proc.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            _say(f"  still compiling {name}.cu ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise BuildError(f"nvcc failed on {name}.cu:\n{log}")
    os.replace(tmp, out)
    for stale in out.parent.glob(f"{stem}.*.so"):          # libraries of earlier versions of this source
        if stale != out and ".tmp" not in stale.name and stale.name.count(".") == out.name.count("."):
            try:
                stale.unlink()
            except OSError:
                pass
    _say(f"built {out.name} in {time.time() - t0:.1f} s")
    return out


# ---- host-only C++ (no CUDA): csrc/host/<name>.cpp ------------------------------------------------
HOST_SOURCES = ("cache_core",)
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC"]


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++)")


def host_library_path(name: str) -> Path:
    src = CSRC / "host" / f"{name}.cpp"
    if not src.is_file():
        raise BuildError(f"no C++ source {src}")
    h = hashlib.sha256(src.read_bytes())
    h.update(" ".join(HOST_FLAGS).encode())
    fname = f"host_{name}.{h.hexdigest()[:12]}.so"
    for d in _build_dirs():
        if (d / fname).is_file():
            return d / fname
    last = None
    for d in _build_dirs():
        try:
            d.mkdir(parents=True, exist_ok=True)
            if not os.access(d, os.W_OK):
                continue
            out = d / fname
            tmp = out.with_suffix(f".tmp{os.getpid()}.so")
            _say(f"compiling host/{name}.cpp ...")
            proc = subprocess.run([find_cxx()] + HOST_FLAGS + ["-o", str(tmp), str(src)], capture_output=True, text=True)
            if proc.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise BuildError(f"C++ compiler failed on host/{name}.cpp:\n{proc.stdout}{proc.stderr}")
            os.replace(tmp, out)
            for stale in d.glob(f"host_{name}.*.so"):
                if stale != out and ".tmp" not in stale.name:
                    try:
                        stale.unlink()
                    except OSError:
                        pass
            return out
        except (OSError, BuildError) as e:
            last = e
    raise BuildError(f"could not build host/{name}.cpp: {last}")


def load_host(name: str) -> ctypes.CDLL:
    key = ("host", name)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(str(host_library_path(name)))
            _loaded[key] = lib
        return lib


def load(name: str, defines=None) -> ctypes.CDLL:
    key = (name, _variant(defines))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(str(library_path(name, defines)))
            _loaded[key] = lib
        return lib


def build_all(names=SOURCES) -> dict:
    """Build every library (cross-compiles without a GPU).  Returns name -> path."""
    out = {n: library_path(n) for n in names if (CSRC / f"{n}.cu").is_file()}
    for n, variants in VARIANTS.items():
        for d in variants:
            out[f"{n}.{_variant(d)}"] = library_path(n, d)
    for n in HOST_SOURCES:
        out[f"host/{n}"] = host_library_path(n)
    return out
