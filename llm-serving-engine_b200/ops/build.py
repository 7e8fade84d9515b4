"""Compile and load the CUDA code of the engine for sm_100a.

Two kinds of binary, both built into ``_build/`` inside the package (or, if that folder cannot be
written, into a per-user folder under the system's temporary directory):

* the core extension (``csrc/binding.cpp`` + the generic ``.cu`` files), built with
  ``torch.utils.cpp_extension.load``;
* one attention library per head size (``csrc/attention.cu`` with ``-DLSE_HEAD_DIM=D``), built
  with a direct ``nvcc`` call and loaded by the core extension.

A build folder's name carries a hash of the sources and flags, so a stale binary is never loaded.
While a compilation runs, a line is printed to stderr every few seconds.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr"]
CORE_CU = ["pointwise.cu", "gemm_f32.cu", "gemm_bf16_tc.cu", "sampling.cu"]
CORE_HEADERS = ["common.cuh", "kernels.h", "attention_args.h", "status.h", "tma_util.cuh", "attention_tc.cuh"]

_core = None
_attn_paths: dict[int, str] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _hash(files: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()[:12]


def build_root() -> Path:
    override = os.environ.get("LLMSERVE_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC.parent / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"llmserve_b200_build_{os.getuid()}")
    for c in candidates:
        try:
            c.mkdir(parents=True, exist_ok=True)
            probe = c / f".w{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return c
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {candidates}")


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"
    exe = Path(cuda_home) / "bin" / "nvcc"
    if exe.exists():
        return str(exe)
    found = shutil.which("nvcc")
    if not found:
        raise BuildError("nvcc not found (set CUDA_HOME); the engine cannot build its kernels")
    return found


def _prune(root: Path, prefix: str, keep: str) -> None:
    """Remove build folders of older source versions (same prefix, another hash)."""
    for d in root.glob(prefix + "*"):
        if d.is_dir() and d.name != keep:
            shutil.rmtree(d, ignore_errors=True)


class _Progress:
    """Prints a line now and then while a compilation runs."""

    def __init__(self, what: str, every: float = 10.0) -> None:
        self.what, self.every = what, every
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        t0 = time.monotonic()
        while not self._stop.wait(self.every):
            print(f"[llmserve_b200] still compiling {self.what} ({time.monotonic() - t0:.0f} s)",
                  file=sys.stderr, flush=True)

    def __enter__(self):
        print(f"[llmserve_b200] compiling {self.what} for sm_100a ...", file=sys.stderr, flush=True)
        self._t0 = time.monotonic()
        self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._t.join()
        if exc[0] is None:
            print(f"[llmserve_b200] compiled {self.what} in {time.monotonic() - self._t0:.0f} s",
                  file=sys.stderr, flush=True)


def load_core(verbose: bool = False):
    """Build (if needed) and import the core extension."""
    global _core
    with _lock:
        if _core is not None:
            return _core
        import torch  # noqa: F401  (the extension links against it)
        from torch.utils import cpp_extension

        sources = [CSRC / "binding.cpp"] + [CSRC / f for f in CORE_CU]
        headers = [CSRC / f for f in CORE_HEADERS]
        tag = _hash(sources + headers, " ".join(ARCH_FLAGS + NVCC_FLAGS) + torch.__version__)
        name = f"lse_core_{tag}"
        folder = build_root() / name
        _prune(build_root(), "lse_core_", name)
        folder.mkdir(parents=True, exist_ok=True)
        # ninja and nvcc must be found even when PATH is minimal
        os.environ["PATH"] = os.pathsep.join(
            [str(Path(sys.executable).parent), str(Path(_nvcc()).parent), os.environ.get("PATH", "")]
        )
        os.environ.setdefault("CUDA_HOME", str(Path(_nvcc()).parent.parent))
        os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 1)))
        built = (folder / f"{name}.so").exists()
        try:
            if built:
                mod = _import_so(folder / f"{name}.so", name)
            else:
                with _Progress("the core kernels"):
                    mod = cpp_extension.load(
                        name=name,
                        sources=[str(s) for s in sources],
                        extra_include_paths=[str(CSRC)],
                        extra_cflags=["-O2", "-std=c++17"],
                        extra_cuda_cflags=ARCH_FLAGS + NVCC_FLAGS,
                        extra_ldflags=["-ldl"],
                        build_directory=str(folder),
                        with_cuda=True,
                        verbose=verbose,
                    )
        except Exception as e:  # noqa: BLE001
            raise BuildError(f"building the core CUDA extension failed: {e}") from e
        _core = mod
        return mod


def _import_so(path: Path, name: str):
    import importlib.util

    import torch  # noqa: F401

    spec = importlib.util.spec_from_file_location(name, str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def attention_library(head_dim: int) -> str:
    """Path of the attention library for ``head_dim``, compiling it if it is not there yet."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise ValueError(
            f"head size {head_dim} is not supported: attention kernels exist for multiples of 16 "
            f"from 16 to 256"
        )
    with _lock:
        if head_dim in _attn_paths:
            return _attn_paths[head_dim]
        src = CSRC / "attention.cu"
        headers = [CSRC / f for f in CORE_HEADERS]
        tag = _hash([src] + headers, " ".join(ARCH_FLAGS + NVCC_FLAGS) + f"D{head_dim}")
        folder = build_root() / f"lse_attn_d{head_dim}_{tag}"
        _prune(build_root(), f"lse_attn_d{head_dim}_", folder.name)
        folder.mkdir(parents=True, exist_ok=True)
        so = folder / f"liblse_attn_d{head_dim}.so"
        if not so.exists():
            tmp = folder / f".tmp{os.getpid()}.so"
            cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, f"-DLSE_HEAD_DIM={head_dim}", "-shared",
                   "-Xcompiler", "-fPIC", f"-I{CSRC}", str(src), "-o", str(tmp)]
            with _Progress(f"attention kernels for head size {head_dim}"):
                r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise BuildError(f"nvcc failed for head size {head_dim}:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, so)
        _attn_paths[head_dim] = str(so)
        return str(so)


def build_all(head_dims=(16, 32, 64, 128), verbose: bool = False) -> None:
    """Compile everything ahead of time (cross-compiles without a GPU)."""
    load_core(verbose=verbose)
    for d in head_dims:
        attention_library(d)
