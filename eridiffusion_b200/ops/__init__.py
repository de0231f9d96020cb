from . import functional, reference  # noqa: F401
