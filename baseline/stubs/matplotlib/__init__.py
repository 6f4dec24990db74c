"""Import stand-in for matplotlib, which this image does not have.

The reference's ``pipeline.py`` imports ``scripts.visualize`` at module level, and that module imports
matplotlib even when no plot is requested. The benchmark's reference arm never asks for plots, so the
names only have to exist; any attempt to draw raises."""
rcParams = {}


def use(*_args, **_kwargs):
    return None


def __getattr__(name):
    raise AttributeError(f"matplotlib stand-in: '{name}' is not available (no plotting in the reference arm)")
