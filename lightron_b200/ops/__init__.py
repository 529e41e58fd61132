from . import functional, native, reference  # noqa: F401
