"""The kernel-module contract of the registry (mirrors tirx_kernels/_protocol.py:12-67).

A kernel module lives at ``tirx_kernels/<category>/.../<module>.py`` and exposes:

``KERNEL_META``
    a *literal* dict assigned exactly once: ``name`` (str, the public ``--kernel`` name),
    ``category`` (str, the containing bucket directory) and ``compute_capability`` (int,
    10 for sm_100a).
``CONFIGS`` / optional ``BENCH_CONFIGS``
    lists of dicts, each with a unique ``label`` plus the keyword arguments of the module's
    functions.  The bench CLI prefers ``BENCH_CONFIGS``.
``get_kernel(**cfg)``
    in the reference, the pre-lowering TIRx function; here, a `KernelHandle` naming the
    C-ABI entry point and the launch arguments derived from the config.
``prepare_data(**cfg)``
    deterministic inputs for one config.
``run_test(**cfg)``
    launch + check; raises ``AssertionError`` (or ``unittest.SkipTest``).
``prepare_bench(**cfg)`` -> object with ``run_gpu(warmup=, repeat=, timer=, rounds=, cooldown_s=)``
    two-stage benchmark entry used by the runner; ``run_bench`` is the one-shot form.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Protocol, runtime_checkable


@dataclass(frozen=True)
class KernelHandle:
    """What `get_kernel` returns in this build: the native entry point for one config."""

    symbol: str
    config: dict[str, Any] = field(default_factory=dict)


@runtime_checkable
class KernelModule(Protocol):
    KERNEL_META: dict[str, Any]
    CONFIGS: list[dict[str, Any]]

    @staticmethod
    def get_kernel(**kwargs: Any) -> Any: ...

    @staticmethod
    def prepare_data(**kwargs: Any) -> Any: ...

    @staticmethod
    def run_test(**kwargs: Any) -> None: ...
