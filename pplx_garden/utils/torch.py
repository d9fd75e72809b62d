"""torch glue: capability probes, profiling ranges, stream helper, module hooks for NVTX /
logging / activation capture, dtype names and memory info.

Covers the helper surface of the reference's python/pplx_garden/utils/torch.py:21-404.
"""

from __future__ import annotations

import dataclasses
import functools
import gc
import os
from contextlib import ContextDecorator, contextmanager
from pathlib import Path
from typing import Any, Callable, Generic, Iterator, Optional, TypeVar

import torch

from pplx_garden.utils import logging_utils

logger = logging_utils.get_logger(__name__)

T = TypeVar("T")
TModule = TypeVar("TModule", bound=torch.nn.Module)


# ---------------------------------------------------------------------------
# clean-up helpers
# ---------------------------------------------------------------------------

def _release_memory() -> None:
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


@contextmanager
def cleanup_context() -> Iterator[None]:
    """Collect garbage and drop cached CUDA blocks when the block ends."""
    try:
        yield
    finally:
        _release_memory()


def cleanup(fn: Callable[..., T]) -> Callable[..., T]:
    """Decorator form of :func:`cleanup_context`."""

    @functools.wraps(fn)
    def wrapper(*args: Any, **kwargs: Any) -> T:
        with cleanup_context():
            return fn(*args, **kwargs)

    return wrapper


# ---------------------------------------------------------------------------
# capability probes
# ---------------------------------------------------------------------------

def has_cuda() -> bool:
    return torch.cuda.is_available() and torch.cuda.device_count() > 0


def has_fp8() -> bool:
    """fp8 tensor-core support: Ada / Hopper / Blackwell (compute capability >= 8.9)."""
    if not has_cuda():
        return False
    major, minor = torch.cuda.get_device_capability()
    return (major, minor) >= (8, 9)


def has_tp(tp: int) -> bool:
    """True when at least ``tp`` GPUs are visible."""
    return has_cuda() and torch.cuda.device_count() >= tp


def has_triton_interpreter() -> bool:
    return os.environ.get("TRITON_INTERPRET", "0") == "1"


def is_blackwell(device: Optional[torch.device] = None) -> bool:
    if not has_cuda():
        return False
    return torch.cuda.get_device_capability(device)[0] == 10


# ---------------------------------------------------------------------------
# profiling
# ---------------------------------------------------------------------------

@contextmanager
def profile_range(name: str) -> Iterator[None]:
    """A range visible both to NVTX consumers and to the torch profiler."""
    if has_cuda():
        torch.cuda.nvtx.range_push(name)
    try:
        with torch.profiler.record_function(name):
            yield
    finally:
        if has_cuda():
            torch.cuda.nvtx.range_pop()


@contextmanager
def capture_profile(trace_file: Optional[Path]) -> Iterator[None]:
    """Record a Chrome trace of the block into ``trace_file`` (no-op when None)."""
    if trace_file is None:
        yield
        return
    activities = [torch.profiler.ProfilerActivity.CPU]
    if has_cuda():
        activities.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(activities=activities, record_shapes=True) as prof:
        yield
    prof.export_chrome_trace(str(trace_file))


def add_nvtx(module: torch.nn.Module, name: Optional[str] = None) -> None:
    """Wrap every forward of ``module`` in an NVTX range."""
    label = name or type(module).__name__

    def before(_mod: torch.nn.Module, _args: Any) -> None:
        torch.cuda.nvtx.range_push(label)

    def after(_mod: torch.nn.Module, _args: Any, _out: Any) -> None:
        torch.cuda.nvtx.range_pop()

    module.register_forward_pre_hook(before)
    module.register_forward_hook(after)


def _walk(module: torch.nn.Module, prefix: str = "") -> Iterator[tuple[str, torch.nn.Module]]:
    yield prefix or type(module).__name__, module
    for child_name, child in module.named_children():
        yield from _walk(child, f"{prefix}.{child_name}" if prefix else child_name)


def _tensors_of(io: Any) -> list[torch.Tensor]:
    if isinstance(io, torch.Tensor):
        return [io]
    if isinstance(io, (list, tuple)):
        return [t for item in io for t in _tensors_of(item)]
    if isinstance(io, dict):
        return [t for item in io.values() for t in _tensors_of(item)]
    return []


def copy_layer_io(io: Any) -> list[torch.Tensor]:
    """Detached CPU copies of every tensor found in a (nested) layer input/output."""
    return [t.detach().to("cpu", copy=True) for t in _tensors_of(io)]


def add_logger(module: torch.nn.Module, log: Optional[Callable[[str], None]] = None) -> None:
    """Log shape/dtype/mean/absmax of every submodule output (debug aid)."""
    emit = log or logger.info

    for name, sub in _walk(module):
        def hook(_m: torch.nn.Module, _a: Any, out: Any, name: str = name) -> None:
            for i, t in enumerate(_tensors_of(out)):
                f = t.detach().float()
                emit(f"{name}[{i}] shape={tuple(t.shape)} dtype={t.dtype} "
                     f"mean={f.mean().item():.6f} absmax={f.abs().max().item():.6f}")

        sub.register_forward_hook(hook)


@dataclasses.dataclass(frozen=True)
class CapturedLayer:
    name: str
    inputs: list[torch.Tensor]
    outputs: list[torch.Tensor]


@dataclasses.dataclass(frozen=True)
class CapturedActivations:
    layers: list[CapturedLayer]
    handles: list[Any]

    def cleanup(self) -> None:
        for h in self.handles:
            h.remove()
        self.handles.clear()


def capture_layer_io(module: torch.nn.Module, layer_names: Optional[set[str]] = None) -> CapturedActivations:
    """Record inputs and outputs of (selected) submodules on every forward."""
    layers: list[CapturedLayer] = []
    handles: list[Any] = []
    for name, sub in _walk(module):
        if layer_names is not None and name not in layer_names:
            continue

        def hook(_m: torch.nn.Module, args: Any, out: Any, name: str = name) -> None:
            layers.append(CapturedLayer(name, copy_layer_io(args), copy_layer_io(out)))

        handles.append(sub.register_forward_hook(hook))
    return CapturedActivations(layers, handles)


def capture_model_activations(model: torch.nn.Module, run: Callable[[], Any],
                              layer_names: Optional[set[str]] = None) -> list[CapturedLayer]:
    """Run ``run()`` once with capture hooks installed and return what was recorded."""
    captured = capture_layer_io(model, layer_names)
    try:
        run()
    finally:
        captured.cleanup()
    return captured.layers


def format_activations_diff(name: str, ref: torch.Tensor, got: torch.Tensor,
                            atol: float = 1e-2, rtol: float = 1e-2) -> str:
    """One-line numeric comparison: cosine similarity, SNR, tolerance violations, error moments."""
    a = ref.detach().float().flatten()
    b = got.detach().float().flatten()
    diff = (a - b).abs()
    cos = torch.nn.functional.cosine_similarity(a, b, dim=0).item() if a.numel() else 1.0
    noise = diff.pow(2).mean().clamp_min(1e-30)
    snr = (10 * torch.log10(a.pow(2).mean().clamp_min(1e-30) / noise)).item() if a.numel() else float("inf")
    atol_pct = 100.0 * (diff > atol).float().mean().item() if a.numel() else 0.0
    rtol_pct = 100.0 * (diff > rtol * a.abs()).float().mean().item() if a.numel() else 0.0
    return (f"{name}: COS: {cos:.4f} SNR: {snr:.2f} ATOL: {atol_pct:.1f}% RTOL: {rtol_pct:.1f}% "
            f"Avg: {diff.mean().item():.6f} Max: {diff.max().item():.6f} Std: {diff.std().item() if diff.numel() > 1 else 0.0:.6f}")


# ---------------------------------------------------------------------------
# dtypes, streams, memory
# ---------------------------------------------------------------------------

def str_to_dtype(dtype: str) -> torch.dtype:
    value = getattr(torch, dtype, None)
    if not isinstance(value, torch.dtype):
        raise ValueError(f"unknown torch dtype {dtype!r}")
    return value


_DTYPE_NAMES = {
    torch.int8: "INT8",
    torch.float8_e4m3fn: "FP8",
    torch.bfloat16: "BFP16",
    torch.float16: "FP16",
    torch.float32: "FP32",
}


def type_to_str(ty: torch.dtype) -> str:
    try:
        return _DTYPE_NAMES[ty]
    except KeyError:
        raise ValueError(f"Unsupported dtype {ty}") from None


class stream_context(ContextDecorator):
    """Run the block on a fresh side stream and make the current stream wait for it.
    On CPU devices (or ``None``) the context does nothing, so CPU-only tests can share code."""

    def __init__(self, device: Optional[torch.device]) -> None:
        self._stream = None
        if device is not None and torch.device(device).type == "cuda":
            self._stream = torch.cuda.Stream(device=device)
        self._guard: Any = None

    def __enter__(self) -> "stream_context":
        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
            self._guard = torch.cuda.stream(self._stream)
            self._guard.__enter__()
        return self

    def __exit__(self, *exc: Any) -> bool:
        if self._stream is not None:
            self._guard.__exit__(*exc)
            torch.cuda.current_stream().wait_stream(self._stream)
        return False


def get_mem_info(device: torch.device) -> tuple[int, int]:
    """(free, total) bytes on the device after dropping caches; (0, 0) for CPU."""
    gc.collect()
    if torch.device(device).type == "cpu":
        return 0, 0
    torch.cuda.empty_cache()
    free, total = torch.cuda.mem_get_info(device)
    return free, total


def get_available_mem(device: torch.device) -> int:
    return get_mem_info(device)[0]


def is_weak_contiguous(inp: torch.Tensor) -> bool:
    """Contiguous, or a permutation that still covers its storage densely."""
    if inp.is_contiguous():
        return True
    storage_bytes = inp.untyped_storage().nbytes() - inp.storage_offset() * inp.element_size()
    return storage_bytes == inp.numel() * inp.element_size()


@contextmanager
def set_default_dtype(dtype: torch.dtype) -> Iterator[None]:
    previous = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        yield
    finally:
        torch.set_default_dtype(previous)


class BorrowedModule(Generic[TModule]):
    """Non-owning reference to a module: holding one inside another ``nn.Module`` does not
    register it as a child (its parameters stay out of ``parameters()`` / ``state_dict()``)."""

    def __init__(self, module: TModule) -> None:
        self.module = module
