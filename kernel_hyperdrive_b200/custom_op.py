"""Registration of the operators as `torch.library` custom ops with an eager bypass.

Mirrors the behaviour of the reference's `cute_op` decorator (cute_kernels/utils/custom_op.py:7-47): in
eager mode the plain Python function runs; while `torch.compile` is tracing, or after
`set_cute_tracing(True)`, the registered custom op is called instead so that the graph holds one opaque
node per kernel launch.  Ops live in the `b200moe::` namespace, so the reference package can be imported
beside this one.
"""

from __future__ import annotations

import inspect
from typing import Callable, Iterable, Sequence

import torch

LIBRARY_NAME = "b200moe"
_IS_TRACING = False


def set_cute_tracing(enable: bool) -> None:
    global _IS_TRACING
    _IS_TRACING = enable


def is_tracing() -> bool:
    return _IS_TRACING or torch.compiler.is_compiling()


def b200_op(name: str, mutates_args: str | Iterable[str] = (), fake_func: Callable | None = None, device_types: str | Sequence[str] | None = "cuda") -> Callable:
    def _inner(func: Callable):
        op = torch.library.custom_op(f"{LIBRARY_NAME}::{name}", func, mutates_args=mutates_args, device_types=device_types)
        if fake_func is not None:
            op.register_fake(fake_func)

        def _run(*args, **kwargs):
            if is_tracing():
                return op(*args, **kwargs)
            return func(*args, **kwargs)

        _run.__signature__ = inspect.signature(func)
        _run.__name__ = func.__name__
        _run.__doc__ = func.__doc__
        _run.custom_op = op
        return _run

    return _inner
