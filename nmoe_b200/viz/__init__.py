"""Read-only run dashboard (HTTP API + one static page) over the metric files."""
from .server import MetricStore, lttb, serve  # noqa: F401
