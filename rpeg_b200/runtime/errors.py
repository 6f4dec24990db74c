"""Exception types of the runtime; the CLIs turn any of them into exit code 2
(reference: RPEG/runtime/errors.py, RPEG/runtime/run.py:87-89)."""


class RuntimeConfigError(ValueError):
    """A run file, plan file or option is invalid or inconsistent."""


class RuntimeDependencyError(RuntimeError):
    """Something the chosen backend needs (CUDA device, native library, NCCL) is unavailable."""


class RuntimeExecutionError(RuntimeError):
    """A graph node failed, timed out or a worker was lost; eligible for bounded replay."""
