"""Durable training state: interval and final checkpoints, their index, the weight-version manifest
and the flat-shard tensor format.

Layout under ``checkpoints.output_dir``::

    checkpoint_index.json                      rpeg.checkpoint_index.v1
    step_<N>/ or final/
        rpeg_weight_versions.json              rpeg.weight_version_checkpoint.v1
        <worker or vertex id>/
            meta.json                          rpeg.flat_shard_checkpoint.v1: tensors, dtypes, byte ranges, sha256
            rank<r>.bin                        the rank's flat shards, back to back, 256-byte aligned

A checkpoint holds, per trainable model, the newest weights with their optimizer state and, when a
model is consumed with positive staleness, every older published version that an unfinished
consumer may still read. Tensors are stored as flat element ranges with their global offsets, so a
run with a different data-parallel degree reloads them by re-slicing (``load_flat_range``).
Reference: RPEG/runtime/algorithms/megatron_ppo_graph.py:3832-3955 (save), :4298-4462 (index and
pruning), :3404-3542 (resume), RPEG/runtime/recovery.md:10-28.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import time
from pathlib import Path
from typing import Any, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

from .errors import RuntimeConfigError, RuntimeExecutionError
from .io import atomic_write_text

INDEX_SCHEMA = "rpeg.checkpoint_index.v1"
VERSIONS_SCHEMA = "rpeg.weight_version_checkpoint.v1"
SHARD_SCHEMA = "rpeg.flat_shard_checkpoint.v1"
INDEX_FILE = "checkpoint_index.json"
VERSIONS_FILE = "rpeg_weight_versions.json"
ALIGN = 256


# ------------------------------------------------------------------------------ index
def load_index(output_dir) -> Dict[str, Any]:
    p = Path(output_dir) / INDEX_FILE
    if not p.exists():
        return {"schema_version": INDEX_SCHEMA, "checkpoints": [], "latest_final": None, "latest_interval": None}
    idx = json.loads(p.read_text())
    if idx.get("schema_version") != INDEX_SCHEMA:
        raise RuntimeConfigError(f"{p} must declare schema_version: {INDEX_SCHEMA}")
    return idx


def entry_path(output_dir, entry: Mapping[str, Any]) -> Path:
    """Directory of an index entry. ``path`` is stored as a path under ``output_dir`` (what the reference's index
    holds); a bare directory name, as older index files of this framework have it, is taken relative to it."""
    p = Path(entry["path"])
    if p.is_absolute() or p.exists():
        return p
    return Path(output_dir) / p.name


def _sort_key(c: Mapping[str, Any]):
    return (int(c["step"]), c["kind"] == "final", str(c["name"]))


def register_checkpoint(output_dir, *, name: str, kind: str, step: int, workers: Sequence[str],
                        extra: Optional[Mapping[str, Any]] = None) -> Dict[str, Any]:
    """Add (or replace) an entry and update ``latest_final`` / ``latest_interval`` (paths under ``output_dir``, as in
    the reference's index); atomic. Call it from ONE process of a job (rank 0)."""
    if kind not in ("interval", "final"):
        raise ValueError("checkpoint kind must be 'interval' or 'final'")
    idx = load_index(output_dir)
    path = str(Path(output_dir) / name)
    entry = {"name": name, "kind": kind, "step": int(step), "path": path, "workers": sorted(workers), "created": time.time(),
             **dict(extra or {})}
    idx["checkpoints"] = [c for c in idx["checkpoints"] if c["name"] != name] + [entry]
    idx["checkpoints"].sort(key=_sort_key)
    idx["latest_final" if kind == "final" else "latest_interval"] = path
    atomic_write_text(Path(output_dir) / INDEX_FILE, json.dumps(idx, indent=2))
    return entry


def prune_checkpoints(output_dir, keep_last_interval_steps: Optional[int], current_step: Optional[int] = None) -> List[str]:
    """Keep the newest ``keep_last_interval_steps`` INTERVAL checkpoints and delete the older ones; ``0`` deletes them
    all, ``None`` keeps everything. The setting counts checkpoints, not steps, as in the reference
    (RPEG/runtime/algorithms/megatron_ppo_graph.py:4349-4380); final checkpoints always stay. ``latest_interval`` is
    recomputed afterwards. Returns the removed names. Call it from ONE process of a job (rank 0)."""
    if keep_last_interval_steps is None:
        return []
    keep = max(0, int(keep_last_interval_steps))
    idx = load_index(output_dir)
    intervals = sorted((c for c in idx["checkpoints"] if c["kind"] == "interval"), key=_sort_key)
    doomed = intervals[: max(0, len(intervals) - keep)]
    removed = []
    for c in doomed:
        target = entry_path(output_dir, c)
        if target.is_dir() and target.parent.resolve() == Path(output_dir).resolve():
            shutil.rmtree(target, ignore_errors=True)
        idx["checkpoints"].remove(c)
        removed.append(c["name"])
    if removed:
        left = [c for c in idx["checkpoints"] if c["kind"] == "interval"]
        idx["latest_interval"] = max(left, key=_sort_key)["path"] if left else None
        atomic_write_text(Path(output_dir) / INDEX_FILE, json.dumps(idx, indent=2))
    return removed


def latest_usable_checkpoint(output_dir, *, max_step: Optional[int] = None, verify: bool = True,
                             verify_hashes: bool = False) -> Optional[Dict[str, Any]]:
    """Newest indexed checkpoint (step <= ``max_step``) that can be restored from: every worker directory present with
    the recorded file sizes (and, with ``verify_hashes``, the recorded sha256). An entry without any worker directory
    holds no tensors and is only accepted when it says so itself (``metadata_only``, written by handlers that keep
    no tensor state); damaged or incomplete checkpoints are skipped."""
    idx = load_index(output_dir)
    for c in sorted(idx["checkpoints"], key=_sort_key, reverse=True):
        if max_step is not None and c["step"] > max_step:
            continue
        if not verify:
            return c
        if not c.get("workers") and not c.get("metadata_only"):
            continue
        if not verify_checkpoint(entry_path(output_dir, c), c["workers"], hashes=verify_hashes)["errors"]:
            return c
    return None


def _sha256_of(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 24), b""):
            h.update(block)
    return h.hexdigest()


def verify_checkpoint(path, workers: Iterable[str], hashes: bool = False) -> Dict[str, Any]:
    """File counts and byte sizes of every worker directory against its ``meta.json``; with ``hashes`` also the
    sha256 of every rank file (a damaged file of the right size is otherwise indistinguishable)."""
    path = Path(path)
    errors: List[str] = []
    files = nbytes = 0
    if not (path / VERSIONS_FILE).exists():
        errors.append(f"{path.name}: missing {VERSIONS_FILE}")
    for w in workers:
        meta_p = path / w / "meta.json"
        if not meta_p.exists():
            errors.append(f"{path.name}/{w}: missing meta.json")
            continue
        meta = json.loads(meta_p.read_text())
        if meta.get("schema_version") != SHARD_SCHEMA:
            errors.append(f"{path.name}/{w}: unexpected schema {meta.get('schema_version')}")
            continue
        for f in meta.get("files", ()):
            fp = path / w / f["name"]
            if not fp.exists():
                errors.append(f"{path.name}/{w}: missing {f['name']}")
            elif fp.stat().st_size != int(f["bytes"]):
                errors.append(f"{path.name}/{w}: {f['name']} has {fp.stat().st_size} bytes, expected {f['bytes']}")
            elif hashes and f.get("sha256") and _sha256_of(fp) != f["sha256"]:
                errors.append(f"{path.name}/{w}: {f['name']} does not match its recorded sha256")
            else:
                files += 1
                nbytes += int(f["bytes"])
    return {"errors": errors, "files": files, "bytes": nbytes}


# ------------------------------------------------------------------------------ weight-version manifest
def write_weight_versions(ckpt_dir, *, step: int, latest: Mapping[str, int], retained: Mapping[str, Sequence[int]],
                          tau: Mapping[str, int]) -> Dict[str, Any]:
    """``latest``: model -> newest version; ``retained``: model -> all versions stored (newest plus
    those an unfinished consumer may still need, i.e. ``latest - tau .. latest``)."""
    doc = {"schema_version": VERSIONS_SCHEMA, "step": int(step), "latest": {k: int(v) for k, v in latest.items()},
           "retained": {k: sorted(int(x) for x in v) for k, v in retained.items()}, "tau": {k: int(v) for k, v in tau.items()}}
    atomic_write_text(Path(ckpt_dir) / VERSIONS_FILE, json.dumps(doc, indent=2))
    return doc


def read_weight_versions(ckpt_dir) -> Dict[str, Any]:
    doc = json.loads((Path(ckpt_dir) / VERSIONS_FILE).read_text())
    if doc.get("schema_version") != VERSIONS_SCHEMA:
        raise RuntimeConfigError(f"{VERSIONS_FILE} must declare schema_version: {VERSIONS_SCHEMA}")
    return doc


def versions_needed_after(step: int, tau: int) -> List[int]:
    """Versions a checkpoint written after logical step ``step`` must hold for a model with staleness
    ``tau``: consumers of steps ``step+1 ..`` read ``max(0, s-1-tau)``, so ``step-tau .. step``."""
    return list(range(max(0, step - tau), step + 1))


# ------------------------------------------------------------------------------ flat shards
def _np_view(t):
    import torch
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy(), "bfloat16"
    return t.numpy(), str(t.dtype).replace("torch.", "")


def save_flat_shards(worker_dir, rank: int, world: int, tensors: Mapping[str, Any], *,
                     ranges: Optional[Mapping[str, Tuple[int, int, int]]] = None, extra: Optional[Mapping[str, Any]] = None) -> Dict[str, Any]:
    """Write this rank's tensors to ``rank<r>.bin`` and (rank 0 merges later) ``meta.rank<r>.json``.
    ``ranges[name] = (global_start, global_stop, global_numel)`` marks a tensor as a shard of a longer
    flat array (optimizer state sharded over data-parallel ranks); unlisted tensors are whole."""
    d = Path(worker_dir)
    d.mkdir(parents=True, exist_ok=True)
    fname = f"rank{rank}.bin"
    entries = []
    h = hashlib.sha256()
    off = 0
    tmp = d / (fname + ".tmp")
    with open(tmp, "wb") as f:
        for name, t in tensors.items():
            arr, dtype = _np_view(t)
            pad = (-off) % ALIGN
            if pad:
                f.write(b"\0" * pad)
                h.update(b"\0" * pad)
                off += pad
            raw = arr.tobytes()
            f.write(raw)
            h.update(raw)
            g0, g1, gn = (ranges or {}).get(name, (0, int(t.numel()), int(t.numel())))
            entries.append({"name": name, "dtype": dtype, "shape": list(t.shape), "offset": off, "bytes": len(raw),
                            "global_start": int(g0), "global_stop": int(g1), "global_numel": int(gn)})
            off += len(raw)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, d / fname)
    part = {"rank": rank, "world": world, "file": {"name": fname, "bytes": off, "sha256": h.hexdigest()}, "tensors": entries,
            "extra": dict(extra or {})}
    atomic_write_text(d / f"meta.rank{rank}.json", json.dumps(part))
    return part


def finalize_worker_meta(worker_dir, world: int, extra: Optional[Mapping[str, Any]] = None) -> Dict[str, Any]:
    """Merge the per-rank parts into ``meta.json`` (called by one rank after all have written)."""
    d = Path(worker_dir)
    parts = []
    for r in range(world):
        p = d / f"meta.rank{r}.json"
        if not p.exists():
            raise RuntimeExecutionError(f"checkpoint part of rank {r} is missing in {d}")
        parts.append(json.loads(p.read_text()))
    meta = {"schema_version": SHARD_SCHEMA, "world": world, "files": [p["file"] for p in parts],
            "ranks": [{"rank": p["rank"], "file": p["file"]["name"], "tensors": p["tensors"], "extra": p["extra"]} for p in parts],
            "extra": dict(extra or {})}
    atomic_write_text(d / "meta.json", json.dumps(meta, indent=1))
    for r in range(world):
        os.unlink(d / f"meta.rank{r}.json")
    return meta


def _read_entry(worker_dir: Path, fname: str, e: Mapping[str, Any], lo: int = 0, hi: Optional[int] = None):
    import numpy as np
    import torch
    np_dtype = {"bfloat16": np.int16, "float32": np.float32, "float16": np.float16, "int32": np.int32, "int64": np.int64,
                "float64": np.float64, "uint8": np.uint8, "int16": np.int16, "bool": np.bool_}[e["dtype"]]
    item = np.dtype(np_dtype).itemsize
    n = e["bytes"] // item
    hi = n if hi is None else hi
    arr = np.fromfile(worker_dir / fname, dtype=np_dtype, count=hi - lo, offset=e["offset"] + lo * item)
    t = torch.from_numpy(arr)
    return t.view(torch.bfloat16) if e["dtype"] == "bfloat16" else t


def load_tensor(worker_dir, name: str):
    """A whole (unsharded) tensor by name, from whichever rank file holds it."""
    d = Path(worker_dir)
    meta = json.loads((d / "meta.json").read_text())
    for r in meta["ranks"]:
        for e in r["tensors"]:
            if e["name"] == name and e["global_stop"] - e["global_start"] == e["global_numel"]:
                return _read_entry(d, r["file"], e).reshape(e["shape"])
    raise KeyError(f"{name} is not stored whole in {d}")


def load_flat_range(worker_dir, name: str, start: int, stop: int):
    """Elements ``[start, stop)`` of the flat array ``name``, assembled from the shards of however
    many ranks wrote it: this is what lets a job resume with a different data-parallel degree."""
    import torch
    d = Path(worker_dir)
    meta = json.loads((d / "meta.json").read_text())
    pieces = []
    for r in meta["ranks"]:
        for e in r["tensors"]:
            if e["name"] != name:
                continue
            lo, hi = max(start, e["global_start"]), min(stop, e["global_stop"])
            if lo < hi:
                pieces.append((lo, _read_entry(d, r["file"], e, lo - e["global_start"], hi - e["global_start"])))
    pieces.sort(key=lambda p: p[0])
    at = start
    for lo, piece in pieces:                 # the shards must tile the range: no gap, no overlap
        if lo != at:
            raise RuntimeExecutionError(f"{name}[{start}:{stop}] in {d}: shards {'overlap' if lo < at else 'leave a gap'} at element {min(lo, at)}")
        at = lo + int(piece.numel())
    if at != stop:
        raise RuntimeExecutionError(f"{name}[{start}:{stop}] is only partly present in {d} ({at - start} elements)")
    return torch.cat([p for _, p in pieces]) if len(pieces) != 1 else pieces[0][1]
