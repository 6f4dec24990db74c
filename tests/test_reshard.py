"""CPU tests of the reshard planner: piece rules, rank mapping, transfer plans against the oracle."""
import pytest
import torch

from rpeg_b200.models.llama import LlamaConfig, ParamLayout
from rpeg_b200.parallel.reshard import (Layout, param_shapes, piece_offsets, plan_transfers, rank_pieces, reshard_state_dict,
                                        shard_state_dict, stage_of, tp_pieces)

CFG = LlamaConfig.tiny(n_layers=4, d_model=512, d_ff=1024, n_heads=4, n_kv_heads=4, vocab=1024, qk_norm=True)


def full_params():
    g = torch.Generator().manual_seed(0)
    return {n: torch.randn(s, generator=g).bfloat16() for n, s in param_shapes(CFG).items()}


def test_rank_mapping_and_stage_ownership():
    lay = Layout(dp=2, pp=2, tp=2)
    assert lay.world == 8 and [lay.coords(lay.rank(d, p, t)) for d in range(2) for p in range(2) for t in range(2)] == \
        [(d, p, t) for d in range(2) for p in range(2) for t in range(2)]
    assert lay.rank(1, 0, 1) == 5
    assert stage_of(CFG, "embed", 2) == 0 and stage_of(CFG, "l1.wqkv", 2) == 0 and stage_of(CFG, "l2.wo", 2) == 1
    assert stage_of(CFG, "final_norm", 2) == 1 and stage_of(CFG, "lm_head", 4) == 3
    assert [stage_of(CFG, f"l{i}.wo", 3) for i in range(4)] == [0, 0, 1, 2]          # 4 layers over 3 stages: 2, 1, 1


def test_tp_pieces_tile_every_parameter_exactly():
    for tp in (1, 2):
        for name, (rows, cols) in param_shapes(CFG).items():
            cover = torch.zeros(rows, cols, dtype=torch.int32)
            for t in range(tp):
                for r0, r1, c0, c1 in tp_pieces(CFG, name, (rows, cols), tp, t):
                    cover[r0:r1, c0:c1] += 1
            replicated = name.endswith("norm") or name.startswith("scalar_head")
            assert bool((cover == (tp if replicated else 1)).all()), name
    q = tp_pieces(CFG, "l0.wqkv", param_shapes(CFG)["l0.wqkv"], 2, 1)
    assert q == [(256, 512, 0, 512), (512 + 256, 512 + 512, 0, 512), (1024 + 256, 1024 + 512, 0, 512)]


@pytest.mark.parametrize("src,dst", [(Layout(1, 1, 2), Layout(2, 1, 1)), (Layout(2, 1, 1), Layout(1, 1, 2)), (Layout(1, 2, 2), Layout(2, 1, 2)),
                                     (Layout(2, 2, 1), Layout(1, 1, 4)), (Layout(1, 1, 4), Layout(1, 4, 1))])
def test_transfer_plan_reproduces_the_oracle(src, dst):
    full = full_params()
    shards = shard_state_dict(CFG, full, src)
    want = reshard_state_dict(CFG, shards, src, dst)
    # flat buffers per rank, as the executor lays them out
    src_flat = []
    for r in range(src.world):
        offs, n = piece_offsets(rank_pieces(CFG, src, r))
        buf = torch.zeros(n, dtype=torch.bfloat16)
        for key, off in offs.items():
            p = shards[r][key]
            buf[off:off + p.numel()] = p.reshape(-1)
        src_flat.append(buf)
    plan = plan_transfers(CFG, src, dst)
    for d in range(dst.world):
        offs, n = piece_offsets(rank_pieces(CFG, dst, d))
        buf = torch.zeros(n, dtype=torch.bfloat16)
        for t in (t for t in plan if t.dst_rank == d):
            s = torch.as_strided(src_flat[t.src_rank], (t.rows, t.cols), (t.src_ld, 1), t.src_offset)
            torch.as_strided(buf, (t.rows, t.cols), (t.dst_ld, 1), t.dst_offset).copy_(s)
        for key, off in offs.items():
            p = want[d][key]
            assert torch.equal(buf[off:off + p.numel()].view(p.shape), p), (d, key)
    # replicas are served by the replica with the matching data-parallel index
    if src.dp > 1 and dst.dp == src.dp:
        assert all(src.coords(t.src_rank)[0] == dst.coords(t.dst_rank)[0] for t in plan)


def test_plan_volume_and_locality():
    cfg = LlamaConfig.llama7b()
    plan = plan_transfers(cfg, Layout(1, 1, 2), Layout(2, 1, 1), dst_ranks=[0])
    total = sum(t.nbytes for t in plan)
    assert total == 2 * sum(r * c for r, c in param_shapes(cfg).values())      # a DP rank ends up with the whole model
    local = sum(t.nbytes for t in plan if t.src_rank == 0)
    assert 0.45 < local / total < 0.55                                          # about half of it was already here
