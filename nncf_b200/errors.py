"""Exception types, named after the reference's (src/nncf/errors.py) so that callers can
catch the same classes by name."""


class ValidationError(Exception):
    """Invalid user-provided configuration."""


class InternalError(Exception):
    """A function was used outside its contract (e.g. integer routine with a float mode)."""


class UnsupportedModelError(Exception):
    """The model / tensor layout is not supported by the algorithm."""


class ParameterNotSupportedError(Exception):
    """An option is not available for this backend."""


class InvalidGroupSizeError(Exception):
    """The reduction channel is not divisible by the group size."""


class LibraryNotBuiltError(ImportError):
    """libnncf_b200.so is missing or cannot be loaded: there is no CPU fallback."""
