from .pipe import AMPnetPipe  # noqa: F401

__all__ = ["AMPnetPipe"]
