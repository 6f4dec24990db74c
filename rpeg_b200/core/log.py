"""Logging for the command-line tools: a logger named ``RPEG`` and an optional tee of stdout into
``logs/run_<timestamp>.log`` (reference: RPEG/core/log.py:27-243)."""
from __future__ import annotations

import logging
import os
import sys
import time
from typing import Optional

_LOGGER_NAME = "RPEG"


class _Tee:
    def __init__(self, stream, path: str):
        self.stream = stream
        self.file = open(path, "a", buffering=1)

    def write(self, data: str) -> int:
        self.file.write(data)
        return self.stream.write(data)

    def flush(self) -> None:
        self.file.flush()
        self.stream.flush()

    def isatty(self) -> bool:
        return False

    def close(self) -> None:
        self.file.close()


def init_logging(log_file: Optional[str] = None, debug: bool = False, tee_stdout: bool = True) -> logging.Logger:
    logger = logging.getLogger(_LOGGER_NAME)
    logger.setLevel(logging.DEBUG if debug else logging.INFO)
    if not logger.handlers:
        h = logging.StreamHandler(sys.stdout)
        h.setFormatter(logging.Formatter("%(message)s"))
        logger.addHandler(h)
    if log_file is None and tee_stdout and os.environ.get("RPEG_LOG_DIR"):
        log_file = os.path.join(os.environ["RPEG_LOG_DIR"], f"run_{time.strftime('%Y%m%d_%H%M%S')}.log")
    if log_file:
        os.makedirs(os.path.dirname(os.path.abspath(log_file)), exist_ok=True)
        if not isinstance(sys.stdout, _Tee):
            sys.stdout = _Tee(sys.stdout, log_file)
            for h in logger.handlers:
                if isinstance(h, logging.StreamHandler):
                    h.setStream(sys.stdout)
    return logger


def get_logger() -> logging.Logger:
    return logging.getLogger(_LOGGER_NAME)


def print_run_header(title: str, **fields) -> None:
    bar = "=" * 78
    print(bar)
    print(f" {title}")
    for k, v in fields.items():
        print(f"   {k:<22} {v}")
    print(bar)
