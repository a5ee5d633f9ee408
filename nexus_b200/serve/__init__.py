"""Continuous-batching server over the paged-KV inference engine."""
from .server import Config, Metrics, Request, Result, Server  # noqa: F401
