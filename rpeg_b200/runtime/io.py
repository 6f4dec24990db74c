"""YAML/JSON mapping files with atomic writes and file hashing (reference: RPEG/runtime/io.py)."""
from __future__ import annotations

import hashlib
import json
import os
import tempfile
from pathlib import Path
from typing import Any, Mapping

import yaml

from .errors import RuntimeConfigError


def load_mapping(path) -> dict:
    p = Path(path)
    if not p.exists():
        raise RuntimeConfigError(f"file not found: {p}")
    with open(p) as f:
        data = yaml.safe_load(f) if p.suffix in (".yaml", ".yml") else json.load(f)
    if not isinstance(data, dict):
        raise RuntimeConfigError(f"{p} must contain a mapping at top level")
    return data


def atomic_write_text(path, text: str) -> None:
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=str(p.parent), prefix=p.name + ".", suffix=".tmp")
    try:
        with os.fdopen(fd, "w") as f:
            f.write(text)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, p)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def dump_mapping(data: Mapping[str, Any], path) -> None:
    p = Path(path)
    if p.suffix in (".yaml", ".yml"):
        atomic_write_text(p, yaml.dump(dict(data), default_flow_style=False, sort_keys=False, allow_unicode=True))
    else:
        atomic_write_text(p, json.dumps(data, indent=2) + "\n")


def sha256_file(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()
