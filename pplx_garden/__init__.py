"""pplx_garden for NVIDIA B200: MoE dispatch/combine over NVLink, a transfer engine for
KV pages and weight shards, CUDA virtual-memory helpers, a process-group layer and a
Unigram tokenizer encoder. The native core is ``pplx_garden._native`` (C++/CUDA built for
sm_100a by ``build.py``); ``pplx_garden._rust`` is an alias of it so that code written
against the reference's extension module name (python-ext/src/lib.rs:8-21) keeps working.
"""

import importlib
import sys

__version__ = "0.1.0"


def _load_native():
    try:
        return importlib.import_module("pplx_garden._native")
    except ImportError as exc:  # pragma: no cover - depends on the build state
        raise ImportError(
            "pplx_garden._native is not built. Run `python build.py` in the repository root "
            "(needs nvcc; compiles for sm_100a without a GPU)."
        ) from exc


_native = _load_native()
sys.modules.setdefault("pplx_garden._rust", _native)
