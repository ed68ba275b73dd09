"""Profiling regions, hierarchical timers and run metadata.

``prof_region_begin / prof_region_end`` and the ``ProfRegion`` context manager mark named
ranges for external profilers (NVTX ranges when CUDA is in use, nothing otherwise), as the
reference's profiling layer does for NVTX / roctx / Score-P
(include/lbann/utils/profiling.hpp:31-110, src/utils/profiling.cpp:28-382).  ``TimerMap``
and ``ScopeTimer`` are the hierarchical wall-clock timers that the training algorithms
print at the end of a run (include/lbann/utils/timer_map.hpp:51-75).  ``system_info``
collects what the reference prints at start-up (src/utils/system_info.cpp).
"""
from __future__ import annotations

import os
import platform
import time
from typing import Dict, List, Optional

import torch

_enabled = True
_stack: List[str] = []


def prof_start() -> None:
    global _enabled
    _enabled = True


def prof_stop() -> None:
    global _enabled
    _enabled = False


def _nvtx():
    return torch.cuda.nvtx if torch.cuda.is_available() and torch.cuda.is_initialized() else None


def prof_region_begin(name: str, color: int = 0, sync: bool = False) -> None:
    """Open a named range.  ``sync`` drains the device first so that the range brackets the
    work it names (src/utils/profiling.cpp prof_region_begin)."""
    if not _enabled:
        return
    nv = _nvtx()
    if sync and nv is not None:
        torch.cuda.synchronize()
    _stack.append(name)
    if nv is not None:
        nv.range_push(name)


def prof_region_end(name: str = "", sync: bool = False) -> None:
    if not _enabled or not _stack:
        return
    nv = _nvtx()
    if sync and nv is not None:
        torch.cuda.synchronize()
    top = _stack.pop()
    if name and name != top:
        raise RuntimeError(f"profiling regions are not nested: closing '{name}' inside '{top}'")
    if nv is not None:
        nv.range_pop()


class ProfRegion:
    """``with ProfRegion("forward"):`` - RAII form of the two calls above."""

    def __init__(self, name: str, color: int = 0, sync: bool = False):
        self.name, self.color, self.sync = name, color, sync

    def __enter__(self):
        prof_region_begin(self.name, self.color, self.sync)
        return self

    def __exit__(self, *exc):
        prof_region_end(self.name, self.sync)
        return False


class TimerMap:
    """Tree of named wall-clock timers: ``scope(name)`` times a block under the current
    node; nested scopes become children."""

    def __init__(self, key: str = "root"):
        self.key = key
        self.times: List[float] = []
        self.children: Dict[str, "TimerMap"] = {}
        self._cursor: List["TimerMap"] = [self]

    def child(self, key: str) -> "TimerMap":
        node = self._cursor[-1]
        if key not in node.children:
            node.children[key] = TimerMap(key)
        return node.children[key]

    def scope(self, key: str) -> "ScopeTimer":
        return ScopeTimer(self, key)

    def total(self) -> float:
        return sum(self.times)

    def report(self, indent: int = 0) -> str:
        pad = "  " * indent
        lines = []
        if self.times:
            n = len(self.times)
            lines.append(f"{pad}{self.key}: total {self.total():.6f}s, {n} calls, "
                         f"mean {self.total() / n:.6f}s")
        else:
            lines.append(f"{pad}{self.key}")
        for c in self.children.values():
            lines.append(c.report(indent + 1))
        return "\n".join(lines)


class ScopeTimer:
    def __init__(self, timers: TimerMap, key: str):
        self.timers, self.key = timers, key
        self.node: Optional[TimerMap] = None

    def __enter__(self):
        self.node = self.timers.child(self.key)
        self.timers._cursor.append(self.node)
        self.t0 = time.perf_counter()
        return self.node

    def __exit__(self, *exc):
        self.node.times.append(time.perf_counter() - self.t0)
        self.timers._cursor.pop()
        return False


def system_info() -> Dict[str, object]:
    """Host, software and device description for the start-up banner and run metadata."""
    info: Dict[str, object] = {
        "host": platform.node(), "platform": platform.platform(), "python": platform.python_version(),
        "torch": torch.__version__, "cuda_runtime": torch.version.cuda, "cpus": os.cpu_count(),
        "omp_threads": torch.get_num_threads(),
    }
    if torch.cuda.is_available():
        props = torch.cuda.get_device_properties(0)
        info.update(gpus=torch.cuda.device_count(), gpu_name=props.name,
                    gpu_memory_gb=round(props.total_memory / 2 ** 30, 1),
                    sm_count=props.multi_processor_count,
                    compute_capability=f"{props.major}.{props.minor}")
    else:
        info["gpus"] = 0
    return info
