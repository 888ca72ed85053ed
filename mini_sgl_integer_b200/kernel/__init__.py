from . import fixed_point  # noqa: F401
