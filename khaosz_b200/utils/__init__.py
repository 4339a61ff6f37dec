from .flat_params import FlatParameters
from .trace import enable_tracing, trace_range, tracing_enabled

__all__ = ["FlatParameters", "enable_tracing", "trace_range", "tracing_enabled"]
