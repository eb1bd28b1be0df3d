"""Build and load the in-tree native extension (sm_100a CUDA kernels + C++ builders).

``build()`` compiles every source under ``csrc/`` with
``-gencode arch=compute_100a,code=sm_100a`` into ``csrc/build/_bf_ext.so``.  ``load()`` imports
that shared object; it rebuilds only when the recorded source digest differs, so a built tree
can be copied to a GPU machine and imported there without a compiler run.  On a machine with a
GPU a missing or unloadable extension is an error — there is no silent PyTorch fallback.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
_BUILD = os.path.join(_CSRC, "build")
_NAME = "_bf_ext"
_LOCK = threading.Lock()
_MOD = None

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fopenmp",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fopenmp"]


def _omp_ldflags():
    """Link against the OpenMP runtime that libtorch already loads (the compiler driver here has no
    libgomp.spec, so a bare -fopenmp at link time fails)."""
    import torch

    tl = os.path.join(os.path.dirname(torch.__file__), "lib")
    if os.path.exists(os.path.join(tl, "libgomp.so.1")):
        return ["-L" + tl, "-l:libgomp.so.1"]
    return ["-lgomp"]


def _sources():
    out = []
    for root, _dirs, files in os.walk(_CSRC):
        if os.path.abspath(root).startswith(os.path.abspath(_BUILD)):
            continue
        for f in sorted(files):
            if f.endswith((".cu", ".cpp", ".h", ".cuh")):
                out.append(os.path.join(root, f))
    return sorted(out)


def source_digest() -> str:
    h = hashlib.sha256()
    for p in _sources():
        h.update(os.path.relpath(p, _CSRC).encode())
        with open(p, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(CUDA_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


def _so_path() -> str:
    return os.path.join(_BUILD, _NAME + ".so")


def _digest_path() -> str:
    return os.path.join(_BUILD, _NAME + ".digest")


def is_built() -> bool:
    if not os.path.exists(_so_path()) or not os.path.exists(_digest_path()):
        return False
    with open(_digest_path()) as fh:
        return fh.read().strip() == source_digest()


def build(verbose: bool = False):
    """Compile (if stale) and import the extension."""
    global _MOD
    from torch.utils import cpp_extension

    os.makedirs(_BUILD, exist_ok=True)
    if not is_built():
        srcs = [p for p in _sources() if p.endswith((".cu", ".cpp"))]
        os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
        os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
        cpp_extension.load(
            name=_NAME,
            sources=srcs,
            extra_cflags=CXX_FLAGS,
            extra_cuda_cflags=CUDA_FLAGS,
            extra_ldflags=_omp_ldflags(),
            extra_include_paths=[_CSRC],
            build_directory=_BUILD,
            with_cuda=True,
            is_python_module=True,
            verbose=verbose,
        )
        with open(_digest_path(), "w") as fh:
            fh.write(source_digest())
    return load()


def _import_so():
    spec = importlib.util.spec_from_file_location(_NAME, _so_path())
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[_NAME] = mod
    return mod


def load():
    """Import the built extension, building it first when it is missing or stale."""
    global _MOD
    if _MOD is not None:
        return _TIMED if _EVENTS_ON else _MOD
    with _LOCK:
        if _MOD is not None:
            return _MOD
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        if not is_built():
            if os.environ.get("BF_NO_BUILD") == "1":
                raise RuntimeError(
                    "budgetformer_b200 native extension is not built (csrc/build/_bf_ext.so missing or stale); "
                    "run `python -c 'import __graft_entry__ as g; g.build()'`")
            _MOD = None
            return build()
        _MOD = _import_so()
        return _TIMED if _EVENTS_ON else _MOD


def available() -> bool:
    """True when the extension can be imported without compiling."""
    try:
        return _MOD is not None or is_built()
    except Exception:
        return False


# ---- launch accounting ------------------------------------------------------------------------------
_LAUNCHES = 0


def count_launches(n: int) -> None:
    """Called by the op wrappers with the number of kernels of this package they just launched."""
    global _LAUNCHES
    _LAUNCHES += int(n)


def launch_count() -> int:
    return _LAUNCHES


def reset_launch_count() -> None:
    global _LAUNCHES
    _LAUNCHES = 0


# ---- per-kernel device times (CUDA events around every extension call) ---------------------------------
# ``enable_kernel_events(True)`` makes ``load()`` hand out a proxy that brackets each extension call with two CUDA
# events on the current stream; ``kernel_event_summary()`` resolves them to milliseconds per entry point.  The time of
# a call is what the stream spent between the two markers: its kernels plus, for the device barriers, the wait for the
# slowest rank.  Off by default (two event records per call); used by ``bench.py --kernel_events``.
_EVENTS_ON = False
_EVENT_LOG = []


class _TimedModule:
    def __getattr__(self, name):
        fn = getattr(_MOD, name)
        if not callable(fn):
            return fn

        def timed(*args, **kw):
            import torch
            if not torch.cuda.is_available():
                return fn(*args, **kw)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn(*args, **kw)
            e.record()
            _EVENT_LOG.append((name, s, e))
            return out

        return timed


_TIMED = _TimedModule()


def enable_kernel_events(on: bool = True) -> None:
    global _EVENTS_ON
    _EVENTS_ON = bool(on)
    _EVENT_LOG.clear()


def kernel_event_summary() -> dict:
    """{entry point: (calls, total ms)} since ``enable_kernel_events``; synchronises the device."""
    import torch
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    out = {}
    for name, s, e in _EVENT_LOG:
        calls, ms = out.get(name, (0, 0.0))
        out[name] = (calls + 1, ms + s.elapsed_time(e))
    _EVENT_LOG.clear()
    return out
