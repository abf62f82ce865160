from .profiling import ClockSampler, EventTimer, chrome_trace, trace_range  # noqa: F401
