"""Read-only run dashboard (HTTP API + a dependency-free page) over the metric files, and the single-file report.

``MetricStore``, ``lttb`` and ``serve`` are reachable from here; they are imported on first use so that
``python -m nmoe_b200.viz.server`` does not load its own module twice."""


def __getattr__(name):
  if name in ("MetricStore", "lttb", "serve", "ExperimentsView"):
    from . import server
    return getattr(server, name)
  raise AttributeError(f"module 'nmoe_b200.viz' has no attribute {name!r}")
