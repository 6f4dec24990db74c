"""Weight resharding between parallel layouts: which piece of which parameter lives on which rank under
``(dp, pp, tp)``, the transfer plan between two layouts, a host-side oracle and the device executor.

Layout rules for the Llama-family parameter table (``models.llama.ParamLayout``):
  * tensor parallel: ``wqkv`` is split by heads (each rank takes its query heads, its key heads and its
    value heads: three row ranges), ``w_gate_up`` by rows inside the gate and the up halves, ``wo`` and
    ``w_down`` by columns (input features), ``embed`` / ``lm_head`` by vocabulary rows; norm weights, QK-norm
    weights and scalar heads are replicated;
  * pipeline parallel: layers are split into ``pp`` contiguous stages; the embedding belongs to the first
    stage, the final norm and the heads to the last;
  * data parallel replicas hold identical pieces; a global rank is ``(dp_i * pp + pp_i) * tp + tp_i``.
A *piece* is a rectangle ``(row0, row1, col0, col1)`` of the full parameter. ``plan_transfers`` intersects the
pieces a destination rank needs with the pieces the source ranks hold and picks, among the replicas that hold a
piece, the one whose data-parallel index matches the destination's (spreads the load over the replicas).
``reshard_state_dict`` is the oracle the executor is tested against; ``ReshardExecutor`` moves the bytes with a
strided peer-copy kernel: every destination rank PULLS its rectangles out of the sources' symmetric buffers.
Reference: RPEG/runtime/reshard.py:16-57 (shard dims, rank mapping), :60-156 (reshard_state_dict), :157-336
(routing), :337-458 (stage ownership).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

Rect = Tuple[int, int, int, int]          # row0, row1, col0, col1


@dataclass(frozen=True)
class Layout:
    dp: int = 1
    pp: int = 1
    tp: int = 1

    @property
    def world(self) -> int:
        return self.dp * self.pp * self.tp

    def rank(self, dp_i: int, pp_i: int, tp_i: int) -> int:
        return (dp_i * self.pp + pp_i) * self.tp + tp_i

    def coords(self, rank: int) -> Tuple[int, int, int]:
        tp_i = rank % self.tp
        pp_i = (rank // self.tp) % self.pp
        return rank // (self.tp * self.pp), pp_i, tp_i


def param_shapes(cfg) -> Dict[str, Tuple[int, int]]:
    """Every parameter as a 2-D shape (vectors are ``[1, n]``)."""
    from ..models.llama import ParamLayout
    out = {}
    for name, (_, shape) in ParamLayout(cfg).entries.items():
        out[name] = (shape[0], shape[1]) if len(shape) == 2 else (1, shape[0])
    return out


def layer_index(name: str) -> Optional[int]:
    """``l<i>.<param>`` -> ``i``; None for parameters outside the decoder layers."""
    head, dot, _ = name.partition(".")
    return int(head[1:]) if dot and head[:1] == "l" and head[1:].isdigit() else None


def stage_of(cfg, name: str, pp: int) -> int:
    """Pipeline stage that owns ``name`` (layers split into contiguous, as even as possible, stages)."""
    if name == "embed":
        return 0
    layer = layer_index(name)
    if layer is None:
        return pp - 1
    per, extra = divmod(cfg.n_layers, pp)
    bound = 0
    for s in range(pp):
        bound += per + (1 if s < extra else 0)
        if layer < bound:
            return s
    return pp - 1


def _split(n: int, parts: int, i: int) -> Tuple[int, int]:
    if n % parts:
        raise ValueError(f"{n} is not divisible by {parts}")
    step = n // parts
    return i * step, (i + 1) * step


def tp_pieces(cfg, name: str, shape: Tuple[int, int], tp: int, t: int) -> List[Rect]:
    """Rectangles of the full parameter that tensor-parallel rank ``t`` of ``tp`` holds."""
    rows, cols = shape
    base = name.split(".", 1)[1] if layer_index(name) is not None else name
    if tp == 1 or base.endswith("norm") or base.startswith("scalar_head"):
        return [(0, rows, 0, cols)]
    if base == "wqkv":
        hd = cfg.head_dim
        q0, q1 = _split(cfg.n_heads, tp, t)
        k0, k1 = _split(cfg.n_kv_heads, tp, t)
        kb, vb = cfg.q_width, cfg.q_width + cfg.kv_width
        return [(q0 * hd, q1 * hd, 0, cols), (kb + k0 * hd, kb + k1 * hd, 0, cols), (vb + k0 * hd, vb + k1 * hd, 0, cols)]
    if base == "w_gate_up":
        f0, f1 = _split(cfg.d_ff, tp, t)
        return [(f0, f1, 0, cols), (cfg.d_ff + f0, cfg.d_ff + f1, 0, cols)]
    if base in ("wo", "w_down"):
        c0, c1 = _split(cols, tp, t)
        return [(0, rows, c0, c1)]
    if base in ("embed", "lm_head"):
        r0, r1 = _split(rows, tp, t)
        return [(r0, r1, 0, cols)]
    raise KeyError(f"no sharding rule for parameter {name}")


def rank_pieces(cfg, layout: Layout, rank: int) -> Dict[str, List[Rect]]:
    """All pieces rank ``rank`` holds under ``layout``."""
    _, pp_i, tp_i = layout.coords(rank)
    out: Dict[str, List[Rect]] = {}
    for name, shape in param_shapes(cfg).items():
        if stage_of(cfg, name, layout.pp) == pp_i:
            out[name] = tp_pieces(cfg, name, shape, layout.tp, tp_i)
    return out


def piece_offsets(pieces: Dict[str, List[Rect]], align: int = 64) -> Tuple[Dict[Tuple[str, int], int], int]:
    """Element offset of every piece inside a rank's flat shard buffer (pieces are stored row-major, dense)."""
    off, table = 0, {}
    for name, rects in pieces.items():
        for i, (r0, r1, c0, c1) in enumerate(rects):
            table[(name, i)] = off
            n = (r1 - r0) * (c1 - c0)
            off += (n + align - 1) // align * align
    return table, off


def _intersect(a: Rect, b: Rect) -> Optional[Rect]:
    r0, r1, c0, c1 = max(a[0], b[0]), min(a[1], b[1]), max(a[2], b[2]), min(a[3], b[3])
    return (r0, r1, c0, c1) if r0 < r1 and c0 < c1 else None


@dataclass(frozen=True)
class Transfer:
    name: str
    src_rank: int
    dst_rank: int
    rect: Rect                 # in coordinates of the full parameter
    src_offset: int            # element offset of rect's first element inside the source shard buffer
    src_ld: int                # row pitch (elements) of the source piece
    dst_offset: int
    dst_ld: int

    @property
    def rows(self) -> int:
        return self.rect[1] - self.rect[0]

    @property
    def cols(self) -> int:
        return self.rect[3] - self.rect[2]

    @property
    def nbytes(self) -> int:
        return self.rows * self.cols * 2


def plan_transfers(cfg, src: Layout, dst: Layout, dst_ranks: Optional[Iterable[int]] = None) -> List[Transfer]:
    """Every rectangle each destination rank must fetch, with its location on a source rank."""
    src_pieces = [rank_pieces(cfg, src, r) for r in range(src.world)]
    src_offsets = [piece_offsets(p)[0] for p in src_pieces]
    plan: List[Transfer] = []
    for d in (range(dst.world) if dst_ranks is None else dst_ranks):
        d_dp, _, _ = dst.coords(d)
        pieces = rank_pieces(cfg, dst, d)
        d_off, _ = piece_offsets(pieces)
        for name, rects in pieces.items():
            for di, need in enumerate(rects):
                covered = 0
                want_dp = d_dp % src.dp
                seen = set()                # replicated parameters are held by several source ranks: take one copy
                order = sorted(range(src.world), key=lambda r: (r != d, r))      # a local copy first
                for s in order:
                    if src.coords(s)[0] != want_dp or name not in src_pieces[s]:
                        continue
                    for si, have in enumerate(src_pieces[s][name]):
                        hit = _intersect(need, have)
                        if hit is None or hit in seen:
                            continue
                        seen.add(hit)
                        s_ld, d_ld = have[3] - have[2], need[3] - need[2]
                        plan.append(Transfer(name, s, d, hit,
                                             src_offsets[s][(name, si)] + (hit[0] - have[0]) * s_ld + (hit[2] - have[2]), s_ld,
                                             d_off[(name, di)] + (hit[0] - need[0]) * d_ld + (hit[2] - need[2]), d_ld))
                        covered += (hit[1] - hit[0]) * (hit[3] - hit[2])
                if covered != (need[1] - need[0]) * (need[3] - need[2]):
                    raise ValueError(f"{name}: destination rank {d} piece {need} is covered by {covered} source elements")
    return plan


# ------------------------------------------------------------------------------ host-side oracle
def shard_state_dict(cfg, full: Dict[str, "object"], layout: Layout) -> List[Dict[Tuple[str, int], "object"]]:
    """Cut full parameters (2-D tensors) into every rank's pieces."""
    out = []
    for r in range(layout.world):
        d = {}
        for name, rects in rank_pieces(cfg, layout, r).items():
            t = full[name]
            t2 = t.reshape(1, -1) if t.dim() == 1 else t
            for i, (r0, r1, c0, c1) in enumerate(rects):
                d[(name, i)] = t2[r0:r1, c0:c1].clone()
        out.append(d)
    return out


def reshard_state_dict(cfg, shards: Sequence[Dict[Tuple[str, int], "object"]], src: Layout, dst: Layout):
    """Oracle: rebuild the full parameters from the source shards (first replica) and cut them for ``dst``."""
    import torch
    shapes = param_shapes(cfg)
    full = {}
    for name, (rows, cols) in shapes.items():
        acc = None
        for r in range(src.world):
            if src.coords(r)[0] != 0:
                continue
            rects = rank_pieces(cfg, src, r).get(name)
            if rects is None:
                continue
            for i, (r0, r1, c0, c1) in enumerate(rects):
                piece = shards[r][(name, i)]
                if acc is None:
                    acc = torch.zeros((rows, cols), dtype=piece.dtype)
                acc[r0:r1, c0:c1] = piece
        full[name] = acc
    return shard_state_dict(cfg, full, dst)


# ------------------------------------------------------------------------------ device executor
class ReshardExecutor:
    """Moves weights from a source layout to a destination layout between the GPUs of one node.

    Every rank exposes its source shard buffer in symmetric memory; ``run`` launches, on each destination
    rank, one strided peer-copy kernel per rectangle it needs (pull over NVLink, or a local copy when the
    source is the rank itself), bracketed by device-side flag barriers: sources are complete before anyone
    pulls, and nobody overwrites its source buffer before every peer is done. The plan is computed once."""

    def __init__(self, cfg, src: Layout, dst: Layout, device, group=None):
        import torch
        import torch.distributed as dist
        from .symm import SignalPad, SymmetricBuffer
        self.cfg, self.src, self.dst = cfg, src, dst
        self.device = torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if src.world != self.world or dst.world != self.world:
            raise ValueError(f"both layouts must use all {self.world} ranks")
        sizes = [piece_offsets(rank_pieces(cfg, src, r))[1] for r in range(self.world)]
        self.src_buf = SymmetricBuffer(max(sizes) * 2, self.device, group)
        self.dst_numel = piece_offsets(rank_pieces(cfg, dst, self.rank))[1]
        self.dst_buf = torch.empty(self.dst_numel, dtype=torch.bfloat16, device=self.device)
        self.plan = plan_transfers(cfg, src, dst, dst_ranks=[self.rank])
        self.pad = SignalPad(self.device, group) if self.world > 1 else None
        self.bytes_in = sum(t.nbytes for t in self.plan)
        self.bytes_remote = sum(t.nbytes for t in self.plan if t.src_rank != self.rank)

    def source(self):
        import torch
        return self.src_buf.tensor(torch.bfloat16)

    def _barrier(self, slot: int) -> None:
        import torch
        from ..ops import kernels as K
        from ..ops._lib import check, lib
        if self.world == 1:
            return
        self.pad.epochs[slot] += 1
        check(lib().rpeg_flag_barrier(self.pad.ptr_array(), self.rank, self.world, slot, self.pad.epochs[slot], None, None,
                                      30_000_000_000, K.status_word(self.device).data_ptr(), torch.cuda.current_stream().cuda_stream),
              "rpeg_flag_barrier")

    def run(self) -> None:
        import torch
        from ..ops._lib import check, lib
        stream = torch.cuda.current_stream().cuda_stream
        self._barrier(0)
        base_dst = self.dst_buf.data_ptr()
        for t in self.plan:
            src_ptr = self.src_buf.peer_ptrs[t.src_rank] + 2 * t.src_offset
            check(lib().rpeg_copy2d(src_ptr, t.src_ld * 2, base_dst + 2 * t.dst_offset, t.dst_ld * 2, t.rows, t.cols * 2, stream), "rpeg_copy2d")
        self._barrier(1)

    def close(self) -> None:
        self.src_buf.close()
        if self.pad is not None:
            self.pad.close()
