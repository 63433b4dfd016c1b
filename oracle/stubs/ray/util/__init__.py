from . import scheduling_strategies  # noqa: F401
