from . import gpu, cpu  # noqa: F401
