"""Process-wide runtime configuration (``crates/torsh-core/src/runtime_config.rs:202-623``):
debug level, validation level, monitoring scope, memory tracking, per-operation overrides and presets,
with environment overrides ``TORSH_DEBUG_LEVEL``, ``TORSH_VALIDATION_LEVEL``, ``TORSH_MEMORY_TRACKING``."""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass, field
from enum import IntEnum


class DebugLevel(IntEnum):
    NONE = 0; ESSENTIAL = 1; STANDARD = 2; VERBOSE = 3; PARANOID = 4


class ValidationLevel(IntEnum):
    ESSENTIAL = 0; STANDARD = 1; STRICT = 2; MAXIMUM = 3


class MonitoringScope(IntEnum):
    NONE = 0; MINIMAL = 1; STANDARD = 2; COMPREHENSIVE = 3


@dataclass
class OperationConfig:
    enable_validation: bool | None = None
    enable_metrics: bool | None = None
    timeout_ms: int | None = None


@dataclass
class RuntimeConfig:
    debug_level: DebugLevel = DebugLevel.STANDARD
    validation_level: ValidationLevel = ValidationLevel.STANDARD
    monitoring_scope: MonitoringScope = MonitoringScope.STANDARD
    memory_tracking: bool = False
    panic_on_warnings: bool = False
    detect_nan_inf: bool = False
    kernel_checks: bool = False       # device-side bounds checks that write the status word
    deterministic: bool = False       # fixed algorithm + reduction order for replay diffs
    operation_configs: dict = field(default_factory=dict)

    _global = None
    _lock = threading.Lock()

    @classmethod
    def global_(cls) -> "RuntimeConfig":
        with cls._lock:
            if cls._global is None:
                cfg = cls()
                cfg._apply_env()
                cls._global = cfg
            return cls._global

    def _apply_env(self):
        e = os.environ
        if "TORSH_DEBUG_LEVEL" in e:
            self.debug_level = DebugLevel[e["TORSH_DEBUG_LEVEL"].upper()]
        if "TORSH_VALIDATION_LEVEL" in e:
            self.validation_level = ValidationLevel[e["TORSH_VALIDATION_LEVEL"].upper()]
        if "TORSH_MEMORY_TRACKING" in e:
            self.memory_tracking = e["TORSH_MEMORY_TRACKING"] not in ("0", "false", "")
        if "TORSH_KERNEL_CHECKS" in e:
            self.kernel_checks = e["TORSH_KERNEL_CHECKS"] not in ("0", "false", "")

    @classmethod
    def development(cls):
        return cls(DebugLevel.VERBOSE, ValidationLevel.STRICT, MonitoringScope.COMPREHENSIVE, True, detect_nan_inf=True)

    @classmethod
    def production(cls):
        return cls(DebugLevel.ESSENTIAL, ValidationLevel.ESSENTIAL, MonitoringScope.MINIMAL, False)

    @classmethod
    def testing(cls):
        return cls(DebugLevel.STANDARD, ValidationLevel.MAXIMUM, MonitoringScope.STANDARD, True, panic_on_warnings=True)

    def set_operation_config(self, op: str, cfg: OperationConfig):
        self.operation_configs[op] = cfg

    def should_validate(self, op: str | None = None, level: ValidationLevel = ValidationLevel.STANDARD) -> bool:
        oc = self.operation_configs.get(op)
        if oc is not None and oc.enable_validation is not None:
            return oc.enable_validation
        return self.validation_level >= level

    def should_collect_metrics(self, op: str | None = None) -> bool:
        oc = self.operation_configs.get(op)
        if oc is not None and oc.enable_metrics is not None:
            return oc.enable_metrics
        return self.monitoring_scope >= MonitoringScope.STANDARD
