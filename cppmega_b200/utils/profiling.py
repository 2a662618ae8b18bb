"""Profiling hooks: NVTX ranges, a torch-profiler capture of N training steps (CUDA kernel table +
chrome trace), and the cudaProfilerStart/Stop window used by ``ncu``/``nsys``
(the reference wires the same three mechanisms through its launchers:
scripts/local_gb10_quarter_train.sh:600-649,787-845; cppmega/recipes/run_profiles.py:235-262)."""
from __future__ import annotations

import contextlib
import os
from typing import Callable, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def install_layer_nvtx(model) -> None:
    """Wrap every hybrid layer's forward in an NVTX range named after its kind and number."""
    for key, layer in getattr(model.decoder, "layers", {}).items():
        name = f"layer{int(key) + 1}:{layer.kind}"
        orig = layer.forward

        def wrapped(*a, _orig=orig, _name=name, **kw):
            with nvtx_range(_name):
                return _orig(*a, **kw)

        layer.forward = wrapped


def profile_steps(step_fn: Callable[[int], None], steps: int, out_dir: Optional[str] = None, row_limit: int = 200) -> str:
    """Run ``step_fn(i)`` for ``steps`` iterations under the torch profiler; returns the kernel table
    sorted by device time and writes ``kernel_table.txt`` / ``by_shape.txt`` into ``out_dir``."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True) as prof:
        for i in range(steps):
            step_fn(i)
        torch.cuda.synchronize()
    table = prof.key_averages().table(sort_by="cuda_time_total", row_limit=row_limit, max_name_column_width=90)
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "kernel_table.txt"), "w") as f:
            f.write(table)
        try:      # the same device time split by operand shapes, which identifies the call sites of the glue ops
            by_shape = prof.key_averages(group_by_input_shape=True).table(
                sort_by="self_cuda_time_total", row_limit=150, max_name_column_width=50, max_shapes_column_width=120)
            with open(os.path.join(out_dir, "by_shape.txt"), "w") as f:
                f.write(by_shape)
        except Exception:
            pass
    return table


@contextlib.contextmanager
def cuda_profiler_window(enabled: bool = True):
    """cudaProfilerStart/Stop bracket for ``ncu --profile-from-start off`` / ``nsys -c cudaProfilerApi``."""
    if enabled and torch.cuda.is_available():
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    try:
        yield
    finally:
        if enabled and torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
