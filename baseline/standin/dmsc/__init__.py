"""Stand-in for the third-party ``dmsc`` middleware package that the reference imports for logging and metrics.

The reference (utils/dc.py:67-89) hard-imports ``dmsc==0.1.8``, which is not installable offline.  This module
lives OUTSIDE the unmodified copy of the reference and is put on ``sys.path`` by the reference arm of
``bench.py`` only; it provides the imported names with inert behaviour (loggers that print warnings, errors and, when
``YV_STANDIN_INFO=1``, info lines to stderr with the seconds since start; metrics that count in memory) so that the reference's own training code runs unchanged.  Nothing of the
framework itself imports it.
"""
from __future__ import annotations

import os
import sys
import time
import types

_T0 = time.time()
_INFO = os.environ.get("YV_STANDIN_INFO", "0") == "1"


class _Logger:
    def _emit(self, level, *a, **k):
        if level in ("WARN", "ERROR") or (level == "INFO" and _INFO):
            try:
                sys.stderr.write(f"[dmsc-standin {level} +{time.time() - _T0:.0f}s] " + " ".join(str(x) for x in a) +
                                 (f" {k}" if k else "") + "\n")
                sys.stderr.flush()
            except Exception:
                pass

    def info(self, *a, **k):
        self._emit("INFO", *a, **k)

    def debug(self, *a, **k):
        pass

    def trace(self, *a, **k):
        pass

    def warn(self, *a, **k):
        self._emit("WARN", *a, **k)

    warning = warn

    def error(self, *a, **k):
        self._emit("ERROR", *a, **k)

    critical = error

    def __getattr__(self, name):
        return lambda *a, **k: None


class _Anything:
    """Accepts any construction, attribute access and call; used for names whose behaviour is never exercised."""

    def __init__(self, *a, **k):
        self.__dict__["_kw"] = dict(k)

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        if name in self.__dict__.get("_kw", {}):
            return self._kw[name]
        return _Anything()

    def __call__(self, *a, **k):
        return _Anything()

    def __iter__(self):
        return iter(())

    def __bool__(self):
        return False

    def __float__(self):
        return 0.0

    def __int__(self):
        return 0

    def __hash__(self):
        return id(self)

    def __eq__(self, other):
        return self is other


class _EnumMeta(type):
    def __getattr__(cls, name):
        if name.startswith("__"):
            raise AttributeError(name)
        member = cls.__new__(cls)
        member.__dict__["name"] = name
        setattr(cls, name, member)
        return member


class _EnumLike(metaclass=_EnumMeta):
    def __repr__(self):
        return f"<{type(self).__name__}.{self.__dict__.get('name')}>"

    def __hash__(self):
        return hash((type(self).__name__, self.__dict__.get("name")))

    def __eq__(self, other):
        return type(self) is type(other) and self.__dict__.get("name") == other.__dict__.get("name")


class _Context:
    def __init__(self):
        self.logger = _Logger()

    def __getattr__(self, name):
        return _Anything()


class _App:
    def __init__(self):
        self._ctx = _Context()

    def get_context(self):
        return self._ctx


class DMSCAppBuilder:
    def __getattr__(self, name):
        if name.startswith("with_"):
            return lambda *a, **k: self
        raise AttributeError(name)

    def build(self):
        return _App()


class DMSCLogConfig(_Anything):
    @classmethod
    def default(cls):
        return cls()


class DMSCMetric:
    def __init__(self, config=None):
        self.config, self.value, self.samples = config, 0.0, []

    def inc(self, v=1.0, *a, **k):
        self.value += float(v)

    def set(self, v, *a, **k):
        self.value = float(v)

    def observe(self, v, *a, **k):
        self.samples.append(float(v))

    def __getattr__(self, name):
        return lambda *a, **k: None


DMSCServiceContext = _Context


class DMSCPythonServiceModule:
    def __init__(self, *a, **k):
        pass


class DMSCPythonAsyncServiceModule:
    def __init__(self, *a, **k):
        pass


_ENUMS = {"DMSCHookKind", "DMSCDeviceType", "DMSCDeviceStatus", "DMSCMetricType"}
_THIS = sys.modules[__name__]


def __getattr__(name: str):
    """Every other ``DMSC*`` name resolves to an inert class (enum-like for the known enumerations)."""
    if not name.startswith("DMSC"):
        raise AttributeError(name)
    cls = _EnumMeta(name, (_EnumLike,), {}) if name in _ENUMS else type(name, (_Anything,), {})
    setattr(_THIS, name, cls)
    return cls
