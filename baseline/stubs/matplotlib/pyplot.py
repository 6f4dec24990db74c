"""Empty part of the matplotlib stand-in (see the package docstring)."""


def __getattr__(name):
    raise AttributeError(f"matplotlib stand-in: '{name}' is not available (no plotting in the reference arm)")
