from . import collectives  # noqa: F401
