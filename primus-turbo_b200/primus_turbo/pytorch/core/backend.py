"""Back-end selection surface of the reference, kept importable.

The reference routes every GEMM through a dispatcher that picks among hipBLASLt / CK / AITER / Triton / FlyDSL kernels
(primus_turbo/pytorch/core/backend.py:66-382: `BackendType`, `PrecisionType`, `BackendChoice`, `GlobalBackendManager`).
This build has exactly one implementation per operator (the sm_100a CUDA library), so nothing is dispatched; but training
scripts call `GlobalBackendManager.set_gemm_backend(BackendType.HIPBLASLT)` and the like at start-up, and the operators
pass `default_backend=BackendType.X.value` around.  These names therefore exist with the same call shapes: setters record
what they were given (getters return it, `reset()` forgets it), environment variables are parsed with the reference's
grammar ("FP8:TRITON,other:HIPBLASLT", "autotune"), and no value changes which kernel runs.  A first use of a setter logs
that once.
"""
import os
from dataclasses import dataclass
from enum import Enum, auto
from typing import Dict, Optional

from ...common.constants import (ENV_AUTO_TUNE, ENV_GEMM_BACKEND, ENV_GROUPED_GEMM_BACKEND,
                                 ENV_MOE_DISPATCH_COMBINE_BACKEND)
from ...common.logger import logger

__all__ = ["BackendChoice", "BackendType", "GlobalBackendManager", "PrecisionType"]


class PrecisionType(Enum):
    FP4 = auto()
    FP8 = auto()
    BF16_FP16_FP32 = auto()


class BackendType(Enum):
    """Member names and order of the reference's enum (the values travel as ints through `default_backend`); B200 is this
    build's own single back end."""
    CK = auto()
    HIPBLASLT = auto()
    AITER = auto()
    TRITON = auto()
    DEEP_EP = auto()
    TURBO = auto()
    FLYDSL = auto()
    HIPKITTENS = auto()
    B200 = auto()


@dataclass
class BackendChoice:
    backend: Optional[BackendType] = None
    auto_tune: bool = False


_PRECISIONS = {"FP4": PrecisionType.FP4, "FP8": PrecisionType.FP8, "BF16": PrecisionType.BF16_FP16_FP32,
               "FP16": PrecisionType.BF16_FP16_FP32, "FP32": PrecisionType.BF16_FP16_FP32}


def _parse_choice(name: str) -> BackendChoice:
    name = name.strip().upper()
    if name == "AUTOTUNE":
        return BackendChoice(auto_tune=True)
    return BackendChoice(backend=BackendType[name])     # KeyError for an unknown name, as in the reference


def _parse_env(value: str) -> Dict[PrecisionType, BackendChoice]:
    """'HIPBLASLT' | 'FP8:TRITON,other:HIPBLASLT' | 'autotune' -> per-precision table."""
    table: Dict[PrecisionType, BackendChoice] = {}
    value = value.strip()
    if not value:
        return table
    if ":" not in value:
        choice = _parse_choice(value)
        return {p: choice for p in set(_PRECISIONS.values())}
    other = None
    for item in value.split(","):
        key, _, name = item.partition(":")
        key = key.strip().upper()
        if key == "OTHER":
            other = _parse_choice(name)
        else:
            table[_PRECISIONS[key]] = _parse_choice(name)
    if other is not None:
        for p in set(_PRECISIONS.values()):
            table.setdefault(p, other)
    return table


class GlobalBackendManager:
    _tables: Dict[str, Dict[PrecisionType, BackendChoice]] = {}
    _auto_tune: Optional[bool] = None
    _told = False

    @classmethod
    def _note(cls):
        if not cls._told:
            cls._told = True
            logger.info("back-end selection is accepted and ignored: this build has one sm_100a implementation per operator",
                        once=True)

    @classmethod
    def _set(cls, slot: str, backend, precision, auto_tune: bool):
        cls._note()
        table = dict(cls._tables.get(slot, {}))
        choice = None if backend is None and not auto_tune else BackendChoice(backend=backend, auto_tune=auto_tune)
        for p in ([precision] if precision is not None else list(set(_PRECISIONS.values()))):
            if choice is None:
                table.pop(p, None)
            else:
                table[p] = choice
        cls._tables[slot] = table

    @classmethod
    def _get(cls, slot: str, env: str, precision: PrecisionType) -> Optional[BackendChoice]:
        if precision in cls._tables.get(slot, {}):
            return cls._tables[slot][precision]
        value = os.environ.get(env)
        if value:
            try:
                return _parse_env(value).get(precision)
            except KeyError:
                logger.warning(f"{env}={value!r} names no known back end; ignored", once=True)
        return None

    @classmethod
    def set_gemm_backend(cls, backend: Optional[BackendType] = None, precision: Optional[PrecisionType] = None,
                         auto_tune: bool = False) -> None:
        cls._set("gemm", backend, precision, auto_tune)

    @classmethod
    def set_grouped_gemm_backend(cls, backend: Optional[BackendType] = None, precision: Optional[PrecisionType] = None,
                                 auto_tune: bool = False) -> None:
        cls._set("grouped_gemm", backend, precision, auto_tune)

    @classmethod
    def set_moe_dispatch_combine_backend(cls, backend: Optional[BackendType] = None, precision: Optional[PrecisionType] = None,
                                         auto_tune: bool = False) -> None:
        assert not auto_tune, "auto-tune is not offered for the dispatch / combine back end"
        cls._set("moe_dispatch_combine", backend, precision, False)

    @classmethod
    def set_auto_tune(cls, enabled: Optional[bool]) -> None:
        cls._note()
        cls._auto_tune = enabled

    @classmethod
    def get_gemm_backend(cls, precision: PrecisionType) -> Optional[BackendChoice]:
        return cls._get("gemm", ENV_GEMM_BACKEND, precision)

    @classmethod
    def get_grouped_gemm_backend(cls, precision: PrecisionType) -> Optional[BackendChoice]:
        return cls._get("grouped_gemm", ENV_GROUPED_GEMM_BACKEND, precision)

    @classmethod
    def get_moe_dispatch_combine_backend(cls, precision: PrecisionType) -> Optional[BackendChoice]:
        return cls._get("moe_dispatch_combine", ENV_MOE_DISPATCH_COMBINE_BACKEND, precision)

    @classmethod
    def auto_tune_enabled(cls) -> bool:
        """Always reported as configured; nothing is tuned (there is nothing to choose between)."""
        if cls._auto_tune is not None:
            return bool(cls._auto_tune)
        return os.environ.get(ENV_AUTO_TUNE, "0") == "1"

    @classmethod
    def reset(cls) -> None:
        cls._tables = {}
        cls._auto_tune = None
