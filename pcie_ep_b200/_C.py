"""Build and load the native extension, in-tree, for sm_100a.

The built library lives in ``pcie_ep_b200/_ext/`` next to the sources it was made from (the
directory is ignored by git), so a copy of the working tree carries it along and no per-user
cache is involved.  ``build()`` compiles every translation unit with
``-gencode arch=compute_100a,code=sm_100a``; importing this module loads the library and builds it
first if it is missing or older than its sources.  There is no fallback: if the library cannot be
built or loaded, importing this module raises (counterpart of the reference's JIT loader,
``pcie_ep/_C.py:25-32``, which targets sm_90 only).

Environment:
    PCIE_EP_B200_BUILD_VERBOSE=1   show compiler output
    PCIE_EP_B200_PROFILE=1         build with per-role timing instrumentation in a separate library
"""

from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
from pathlib import Path
from typing import List

_ROOT = Path(__file__).resolve().parents[1]
_CSRC = _ROOT / "csrc"
_PROFILE = os.getenv("PCIE_EP_B200_PROFILE", "0") == "1"
# the instrumented library is built in a directory of its own so that the two builds never share object files
_EXT_DIR = Path(__file__).resolve().parent / "_ext" / "prof" if _PROFILE else Path(__file__).resolve().parent / "_ext"
_NAME = "pcie_ep_b200_cuda_prof" if _PROFILE else "pcie_ep_b200_cuda"

SOURCES: List[Path] = [
    _CSRC / "runtime.cpp",
    _CSRC / "kernels" / "launch.cu",
    _CSRC / "kernels" / "expert_gemm.cu",
    _CSRC / "kernels" / "layout_static.cu",
    _CSRC / "kernels" / "litmus.cu",
]

CUDA_FLAGS = [
    "-O3",
    "-lineinfo",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
]
HOST_FLAGS = ["-O2", "-std=c++17"]
if _PROFILE:
    CUDA_FLAGS.append("-DBEP_ENABLE_PROFILING=1")
    HOST_FLAGS.append("-DBEP_ENABLE_PROFILING=1")


def _existing_sources() -> List[Path]:
    return [path for path in SOURCES if path.exists()]


def source_fingerprint() -> str:
    """Hash of every file the library is built from (sources and headers)."""
    digest = hashlib.sha256()
    files = sorted(p for p in _CSRC.rglob("*") if p.suffix in (".cu", ".cuh", ".cpp", ".hpp", ".h"))
    for path in files:
        digest.update(str(path.relative_to(_CSRC)).encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(CUDA_FLAGS + HOST_FLAGS).encode())
    return digest.hexdigest()


def _library_path() -> Path:
    return _EXT_DIR / f"{_NAME}.so"


def _stamp_path() -> Path:
    return _EXT_DIR / f"{_NAME}.sha256"


def is_built() -> bool:
    return _library_path().exists() and _stamp_path().exists() and _stamp_path().read_text().strip() == source_fingerprint()


def build(verbose: bool = False) -> Path:
    """Compile the extension for sm_100a into ``pcie_ep_b200/_ext`` (no GPU needed)."""
    from torch.utils.cpp_extension import load

    _EXT_DIR.mkdir(parents=True, exist_ok=True)
    # torch would otherwise add -gencode flags from its own arch list; an empty list plus the
    # explicit flag above gives exactly one target: sm_100a.
    previous = os.environ.get("TORCH_CUDA_ARCH_LIST")
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    try:
        load(
            name=_NAME,
            sources=[str(p) for p in _existing_sources()],
            extra_include_paths=[str(_CSRC)],
            extra_cuda_cflags=CUDA_FLAGS,
            extra_cflags=HOST_FLAGS,
            build_directory=str(_EXT_DIR),
            verbose=verbose or bool(int(os.getenv("PCIE_EP_B200_BUILD_VERBOSE", "0"))),
            is_python_module=True,
        )
    finally:
        if previous is None:
            os.environ.pop("TORCH_CUDA_ARCH_LIST", None)
        else:
            os.environ["TORCH_CUDA_ARCH_LIST"] = previous
    _stamp_path().write_text(source_fingerprint())
    return _library_path()


def _load():
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    if not is_built():
        build()
    name = _NAME
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, str(_library_path()))
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot load native extension from {_library_path()}")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[name] = module
    return module


_module = _load()

Runtime = _module.Runtime
HostSegment = _module.HostSegment
NumaRelay = _module.NumaRelay
segment_layout = _module.segment_layout
allocate_device_segment = _module.allocate_device_segment
export_device_segment = _module.export_device_segment
import_device_segment = _module.import_device_segment
release_imported_segment = _module.release_imported_segment
free_device_segment = _module.free_device_segment
get_device_numa_node = _module.get_device_numa_node
query_numa_pages = _module.query_numa_pages
create_host_segment = _module.create_host_segment
first_touch_host_segment = _module.first_touch_host_segment
dispatch_group = _module.dispatch_group
combine_group = _module.combine_group
tensor_refs = _module.tensor_refs


def __getattr__(name: str):
    return getattr(_module, name)
