"""Multi-GPU self test of the peer-memory layer, run with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29551 \
        -m rpeg_b200.parallel.selftest

Checks, each against values computed independently on the host or with NCCL:
  1 symmetric buffers   every rank reads every peer's buffer through its IPC mapping
  2 flag barrier        the payload exchange returns every rank's value; no wait times out
  3 fused DP optimizer  reduce-scatter + Adam + all-gather over peer memory equals AdamW on the summed
                        gradients computed with torch, and all ranks end with identical weights
  4 GRPO steps          two data-parallel steps of the tiny model: finite loss, identical weights
  5 fused GEMM+RS       the row-parallel linear (GEMM with reduce-scatter / all-reduce in one kernel) against
                        an fp32 all-reduce of the partial products, three calls in a row
  6 fused AG+GEMM       the column-parallel linear (all-gather of activation rows + GEMM in one kernel) against
                        fp32, four calls in a row over the two input buffers
  7 reshard             tensor-parallel shards -> data-parallel replicas and back with the strided peer-copy executor,
                        bit-exact against the host-side oracle
  8 TP forward          a two-layer model's token log-probs through the tensor-parallel forward (two all-gather+GEMM and
                        two GEMM+reduce-scatter launches per layer, vocabulary-parallel head) against the plain forward
Rank 0 prints one JSON line with ``"ok": true``. Exit code 1 on any mismatch.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist


def _progress(rank: int, step: str) -> None:
    """One line per step on stderr (rank 0), so that a run that stops shows where."""
    if rank == 0:
        print(f"[selftest] step {step}", file=sys.stderr, flush=True)


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from ..engine import algorithms as A
    from ..engine.optimizer import AdamW
    from ..engine.trainers import GRPOTrainer
    from ..models.llama import LlamaConfig, LlamaModel
    from ..ops import kernels as K
    from ..ops._lib import check, lib
    from .dp import DPContext
    from .symm import SymmetricBuffer, SymmetricMemoryCorruption, check_canaries
    guards: list = []

    def guards_intact(where: str) -> None:
        """Guard bytes around every live symmetric buffer of this rank (a peer's kernel may have written them)."""
        torch.cuda.synchronize()
        dist.barrier()
        try:
            check_canaries()
            guards.append(True)
        except SymmetricMemoryCorruption as exc:
            print(json.dumps({"rank": rank, "where": where, "error": str(exc)}), file=sys.stderr)
            guards.append(False)

    report = {"world": world}
    stream = lambda: torch.cuda.current_stream().cuda_stream

    _progress(rank, "1")
    # 1 symmetric buffers
    buf = SymmetricBuffer(1 << 20, dev)
    buf.tensor(torch.float32).fill_(float(rank + 1))
    torch.cuda.synchronize()
    dist.barrier()
    got = []
    tmp = torch.empty(1 << 18, dtype=torch.float32, device=dev)
    for p in range(world):
        check(lib().rpeg_copy16(buf.peer_ptrs[p], tmp.data_ptr(), 1 << 20, stream()), "rpeg_copy16")
        got.append((float(tmp.min()), float(tmp.max())))
    report["peer_reads_ok"] = got == [(float(p + 1), float(p + 1)) for p in range(world)]
    dist.barrier()

    _progress(rank, "2")
    # 2 flag barrier with payload
    dp = DPContext(dev)
    mine = torch.tensor([10.0 + rank], device=dev)
    out = torch.zeros(K.MAX_PEERS, device=dev)
    for _ in range(3):
        dp.barrier(5, payload_in=mine, payload_out=out)
    K.check_status()
    report["barrier_payload_ok"] = out[:world].tolist() == [10.0 + r for r in range(world)]

    _progress(rank, "3")
    # 3 fused optimizer step against torch AdamW on the summed gradients
    cfg = LlamaConfig.tiny(n_layers=2)
    w = dp.alloc_weights(cfg)
    g = dp.alloc_grads(cfg)
    model = LlamaModel(cfg, dev, trainable=True, weights=w, grads=g, seed=11)
    model.init_weights(11)
    n = model.layout.total
    w0 = model.w[:n].float().clone()
    opt = AdamW(model, lr=1e-2, dp=dp, max_grad_norm=1.0)
    gens = [torch.Generator(device="cpu").manual_seed(100 + r) for r in range(world)]
    ref_p, ref_m, ref_v = w0.clone(), torch.zeros_like(w0), torch.zeros_like(w0)
    ok_steps = []
    for step in range(1, 6):
        grads = [torch.randn(n, generator=gens[r]) * 0.01 for r in range(world)]
        model.g[:n].copy_(grads[rank].to(dev))
        if step >= 4:
            # the same step with the reduction done in per-layer buckets on the side stream, as under a backward pass
            hook = dp.overlap_hook(opt, model, bucket_layers=1)
            for layer in reversed(range(cfg.n_layers)):
                hook(layer)
        opt.step()
        torch.cuda.synchronize()
        K.check_status()
        gsum = torch.stack(grads).sum(0).to(dev)
        norm = gsum.norm()
        gsum = gsum * torch.clamp(1.0 / (norm + 1e-6), max=1.0)
        ref_m = 0.9 * ref_m + 0.1 * gsum
        ref_v = 0.999 * ref_v + 0.001 * gsum * gsum
        ref_p = ref_p - 1e-2 * (ref_m / (1 - 0.9 ** step)) / ((ref_v / (1 - 0.999 ** step)).sqrt() + 1e-8)
        err = (model.w[:n].float() - ref_p.bfloat16().float()).abs().max().item()
        nerr = abs(float(opt.grad_norm()) - float(norm)) / float(norm)
        ok_steps.append(err <= 2e-2 * ref_p.abs().max().item() and nerr < 1e-3)
    report["fused_adam_ok"] = all(ok_steps)
    chk = model.w[:n].float().sum().reshape(1).double()
    lo, hi = chk.clone(), chk.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    report["weights_identical_after_adam"] = bool((lo == hi).item())
    guards_intact("fused data-parallel optimizer step")

    _progress(rank, "4")
    # 4 two GRPO steps, data parallel
    algo = A.AlgoConfig(kl_coef=0.04, micro_tokens=512, head_chunk=256)
    tr = GRPOTrainer(cfg, device=dev, samples_per_prompt=4, max_new=24, prompt_len=16, algo=algo, dp=DPContext(dev), gen_slots=8,
                     kv_budget_bytes=1e9, seed=5, eos_id=1, lr=1e-4)
    gcpu = torch.Generator().manual_seed(77)
    losses = []
    for it in range(2):
        prompts = torch.randint(2, cfg.vocab, (4 * world, 16), generator=gcpu, dtype=torch.int32)
        rewards = torch.randn(16 * world, generator=gcpu)
        outm = tr.step(prompts[rank * 4:(rank + 1) * 4].contiguous(), rewards[rank * 16:(rank + 1) * 16].contiguous())
        losses.append(outm["loss"])
    K.check_status()
    chk = tr.actor.w[: tr.actor.layout.total].float().sum().reshape(1).double()
    lo, hi = chk.clone(), chk.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    report["grpo_losses_finite"] = all(x == x and abs(x) < 1e6 for x in losses)
    report["weights_identical_after_grpo"] = bool((lo == hi).item())

    _progress(rank, "5")
    # 5 fused GEMM + reduce-scatter / all-reduce over peer memory against an fp32 all-reduce of the partial products
    from .tp import RowParallelLinear
    gq = torch.Generator().manual_seed(300 + rank)
    Mrows, Nout, Kp = 256 * world, 1024 + 64, 512 + 64         # N and K not multiples of the tile: edge paths
    wsh = (torch.randn(Nout, Kp, generator=gq) * 0.05).bfloat16().to(dev)
    rs_ok = []
    for all_red in (False, True):
        layer = RowParallelLinear(wsh, max_rows=Mrows, device=dev, all_reduce=all_red)
        for it in range(3):                                     # several epochs on the same counters
            xsh = torch.randn(Mrows, Kp, generator=gq).bfloat16().to(dev)
            y = layer.forward(xsh).float().clone()
            ref = xsh.float() @ wsh.float().t()
            dist.all_reduce(ref)
            if not all_red:
                ref = ref[rank * (Mrows // world):(rank + 1) * (Mrows // world)]
            torch.cuda.synchronize()
            K.check_status()
            rs_ok.append(bool(((y - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-3).item()))
            y2 = layer.forward_unfused(xsh).float()
            rs_ok.append(bool(((y2 - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-3).item()))
        guards_intact("gemm + reduce-scatter")
        layer.close()
    report["fused_gemm_reduce_scatter_ok"] = all(rs_ok)

    _progress(rank, "6")
    # 6 fused all-gather + GEMM (column-parallel linear): every rank contributes its rows, result against fp32
    from .tp import ColumnParallelLinear
    gx = torch.Generator().manual_seed(900)                 # the same activation on every rank; each keeps its rows
    Mrows, Kin, Nloc = 256 * world, 512 + 64, 320
    wcol = (torch.randn(Nloc, Kin, generator=gq) * 0.05).bfloat16().to(dev)
    col = ColumnParallelLinear(wcol, max_rows=Mrows, device=dev)
    ag_ok = []
    per = Mrows // world
    for it in range(4):
        x_full = torch.randn(Mrows, Kin, generator=gx).bfloat16()
        col.input_rows(Mrows).copy_(x_full[rank * per:(rank + 1) * per].to(dev))
        y = col.forward(Mrows).float()
        ref = x_full.to(dev).float() @ wcol.float().t()
        torch.cuda.synchronize()
        K.check_status()
        ag_ok.append(bool(((y - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-3).item()))
        y2 = col.forward_unfused(x_full[rank * per:(rank + 1) * per].to(dev)).float()
        ag_ok.append(bool(((y2 - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-3).item()))
    guards_intact("all-gather + gemm")
    col.close()
    report["fused_all_gather_gemm_ok"] = all(ag_ok)

    _progress(rank, "7")
    # 7 weight reshard TP=world -> DP=world (every rank ends with the whole model) and back, against the host oracle
    from .reshard import Layout, ReshardExecutor, param_shapes, piece_offsets, rank_pieces, shard_state_dict
    rcfg = LlamaConfig.tiny(n_layers=2, d_model=512, d_ff=1024, n_heads=8, n_kv_heads=8, vocab=1024)
    gfull = torch.Generator().manual_seed(4242)
    full = {nm: torch.randn(sh, generator=gfull).bfloat16() for nm, sh in param_shapes(rcfg).items()}
    rs_ok = []
    for src_l, dst_l in ((Layout(1, 1, world), Layout(world, 1, 1)), (Layout(world, 1, 1), Layout(1, 1, world))):
        ex = ReshardExecutor(rcfg, src_l, dst_l, dev)
        mine = shard_state_dict(rcfg, full, src_l)[rank]
        offs, _ = piece_offsets(rank_pieces(rcfg, src_l, rank))
        src_flat = ex.source()
        for key, off in offs.items():
            src_flat[off:off + mine[key].numel()].copy_(mine[key].reshape(-1).to(dev))
        for _ in range(2):
            ex.dst_buf.zero_()
            ex.run()
        torch.cuda.synchronize()
        K.check_status()
        want = shard_state_dict(rcfg, full, dst_l)[rank]
        doffs, _ = piece_offsets(rank_pieces(rcfg, dst_l, rank))
        rs_ok.append(all(torch.equal(ex.dst_buf[o:o + want[k].numel()].cpu().view(want[k].shape), want[k]) for k, o in doffs.items()))
        guards_intact("reshard executor")
        ex.close()
    report["reshard_executor_ok"] = all(rs_ok)

    _progress(rank, "8")
    # 8 tensor-parallel forward (sequence-parallel layers from the fused linears) against the single-GPU forward
    from ..models.tp_llama import TPLlamaForward
    tcfg = LlamaConfig.tiny(n_layers=2, d_model=1024, d_ff=1024, n_heads=8, n_kv_heads=8, vocab=1024)
    tmodel = LlamaModel(tcfg, dev, seed=21)
    lens = [37, 130, 200]
    gt = torch.Generator().manual_seed(5)
    toks = torch.randint(0, tcfg.vocab, (sum(lens),), generator=gt, dtype=torch.int32).to(dev)
    tgts = torch.randint(0, tcfg.vocab, (sum(lens),), generator=gt, dtype=torch.int32).to(dev)
    tpos = torch.cat([torch.arange(l) for l in lens]).to(dev, torch.int32)
    tcu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=dev, dtype=torch.int32)
    xf_ref, _ = tmodel.forward(toks, tpos, tcu, max(lens))
    lp_ref = tmodel.token_logprobs(xf_ref, tgts)
    tp_fwd = TPLlamaForward(tmodel, max_tokens=sum(lens))
    tp_ok = []
    for _ in range(2):
        lp_tp = tp_fwd.token_logprobs(toks, tpos, tcu, max(lens), tgts)
        torch.cuda.synchronize()
        K.check_status()
        tp_ok.append(bool(((lp_tp - lp_ref).abs().max() < 8e-2).item()))
    guards_intact("tensor-parallel forward")
    tp_fwd.close()
    report["tensor_parallel_forward_ok"] = all(tp_ok)

    _progress(rank, "8b")
    # 8b tensor-parallel TRAINING step (fused linears in both directions, vocabulary-parallel loss, sharded AdamW)
    #    against the same step on the whole model
    from ..models.tp_llama import TPAdamW, TPLlamaTrain
    from ..engine.optimizer import AdamW
    from .reshard import param_shapes as _shapes, tp_pieces as _pieces
    wcfg = LlamaConfig.tiny(n_layers=2, d_model=1024, d_ff=1024, n_heads=8, n_kv_heads=8, vocab=1024)
    whole_t = LlamaModel(wcfg, dev, trainable=True, seed=51)
    gq_ = torch.Generator().manual_seed(61)
    Nt, St, Tt = 6, 40, 60
    plt_ = [int(x) for x in torch.randint(8, St + 1, (Nt,), generator=gq_)]
    rlt_ = [int(x) for x in torch.randint(5, Tt + 1, (Nt,), generator=gq_)]
    mask_t = torch.zeros(Nt, Tt)
    for r_, l_ in enumerate(rlt_):
        mask_t[r_, :l_] = 1.0
    ro_t = A.Rollout(prompt_ids=torch.randint(2, wcfg.vocab, (Nt, St), generator=gq_, dtype=torch.int32).to(dev), prompt_lens=plt_,
                     resp_ids=torch.randint(2, wcfg.vocab, (Nt, Tt), generator=gq_, dtype=torch.int32).to(dev), resp_lens=rlt_,
                     old_logp=(-torch.rand(Nt, Tt, generator=gq_) * 3 * mask_t).to(dev), mask=mask_t.to(dev))
    ro_t.ref_logp = (ro_t.old_logp * 1.05).contiguous()
    ro_t.adv = (torch.randn(Nt, Tt, generator=gq_) * mask_t).to(dev)
    talgo = A.AlgoConfig(kl_coef=0.05, micro_tokens=320, head_chunk=256)
    tpm = TPLlamaTrain(whole_t, max_tokens=512)
    want_t = A.policy_train_step(whole_t, ro_t, talgo)
    got_t = A.policy_train_step_tp(tpm, ro_t, talgo)
    tpm.sync_replicated_grads()
    torch.cuda.synchronize()
    K.check_status()
    shapes_t = _shapes(wcfg)
    tpt_ok = [abs(float(got_t["loss"]) - float(want_t["loss"])) < 3e-3 * max(1.0, abs(float(want_t["loss"])))]

    def _piece_of(t_full, name):
        ps = [t_full[r0:r1, c0:c1] for r0, r1, c0, c1 in _pieces(wcfg, name, shapes_t[name], world, rank)]
        return torch.cat(ps, 0) if len(ps) > 1 else ps[0]

    for name in tpm.entries:
        ref_g = whole_t.gp[name].float() if name in tpm.entries and tpm.entries[name][0] < tpm.n_replicated else _piece_of(whole_t.gp[name].float(), name)
        got_g = tpm.gp[name].float()
        tpt_ok.append(bool(((got_g - ref_g).norm() <= 4e-2 * ref_g.norm() + 1e-6).item()))
    opt_w, opt_tp = AdamW(whole_t, lr=1e-3), TPAdamW(tpm, lr=1e-3)
    opt_w.step()
    opt_tp.step(sync_replicated=False)                          # summed above for the comparison
    torch.cuda.synchronize()
    tpt_ok.append(abs(float(opt_w.grad_norm()) - float(opt_tp.grad_norm())) < 4e-2 * float(opt_w.grad_norm()) + 1e-6)
    for name in ("l1.w_down", "l0.wqkv", "lm_head", "final_norm"):
        ref_w = whole_t.p[name].float() if tpm.entries[name][0] < tpm.n_replicated else _piece_of(whole_t.p[name].float(), name)
        tpt_ok.append(bool(((tpm.p[name].float() - ref_w).abs().max() < 4e-3).item()))
    report["tensor_parallel_training_ok"] = all(tpt_ok)
    guards_intact("tensor-parallel training")
    tpm.close()

    _progress(rank, "9")
    # 9 pipeline-parallel policy step (1F1B over all ranks as stages) against the same step on the whole model
    from .pp import PipelineRunner
    pcfg = LlamaConfig.tiny(n_layers=max(2, world), vocab=512)
    whole = LlamaModel(pcfg, dev, trainable=True, seed=33)
    stage_m = LlamaModel(pcfg, dev, trainable=True, seed=1, stage=(rank, world))
    for name in stage_m.layout.entries:
        stage_m.p[name].copy_(whole.p[name])
    gp_ = torch.Generator().manual_seed(91)
    Np, Sp, Tp_ = 8, 12, 20
    pl = [int(x) for x in torch.randint(4, Sp + 1, (Np,), generator=gp_)]
    rl = [int(x) for x in torch.randint(3, Tp_ + 1, (Np,), generator=gp_)]
    mask_p = torch.zeros(Np, Tp_)
    for r_, l_ in enumerate(rl):
        mask_p[r_, :l_] = 1.0
    ro_p = A.Rollout(prompt_ids=torch.randint(2, pcfg.vocab, (Np, Sp), generator=gp_, dtype=torch.int32).to(dev), prompt_lens=pl,
                     resp_ids=torch.randint(2, pcfg.vocab, (Np, Tp_), generator=gp_, dtype=torch.int32).to(dev), resp_lens=rl,
                     old_logp=(-torch.rand(Np, Tp_, generator=gp_) * 3 * mask_p).to(dev), mask=mask_p.to(dev))
    ro_p.ref_logp = (ro_p.old_logp * 1.05).contiguous()
    ro_p.adv = (torch.randn(Np, Tp_, generator=gp_) * mask_p).to(dev)
    palgo = A.AlgoConfig(kl_coef=0.05, micro_tokens=64, head_chunk=64)
    want_m = A.policy_train_step(whole, ro_p, palgo)
    runner = PipelineRunner(stage_m)
    got_m = A.policy_train_step(stage_m, ro_p, palgo, pipeline=runner)
    lp_whole = A.sequence_logprobs(whole, ro_p, palgo)
    lp_pipe = A.sequence_logprobs(stage_m, ro_p, palgo, pipeline=runner)
    torch.cuda.synchronize()
    K.check_status()
    pp_ok = [abs(float(got_m["loss"]) - float(want_m["loss"])) < 2e-3 * max(1.0, abs(float(want_m["loss"]))),
             bool(((lp_whole - lp_pipe).abs().max() < 5e-2).item())]
    for name in stage_m.layout.entries:
        a_, b_ = stage_m.gp[name].float(), whole.gp[name].float()
        pp_ok.append(bool(((a_ - b_).norm() <= 3e-2 * b_.norm() + 1e-6).item()))
    report["pipeline_parallel_ok"] = all(pp_ok)
    report["pipeline_p2p_calls"] = runner.p2p_calls
    dist.barrier()

    _progress(rank, "9b")
    # 9b fused bidirectional actor/critic pipeline: actor stages in rank order, critic stages in reverse order, one
    #    interleaved instruction stream per rank, against the two unfused whole-model steps
    from dataclasses import replace as _replace
    from .fused_pp import FusedPipelineExecutor, logical_stage, uniform_schedule
    fcfg_a = LlamaConfig.tiny(n_layers=max(2, world), vocab=512)
    fcfg_c = _replace(fcfg_a, lm_head=False, scalar_head=True)
    whole_a = LlamaModel(fcfg_a, dev, trainable=True, seed=41)
    whole_c = LlamaModel(fcfg_c, dev, trainable=True, seed=42)
    Nf = 4 * world
    gf = torch.Generator().manual_seed(97)
    plf = [int(x) for x in torch.randint(4, 13, (Nf,), generator=gf)]
    rlf = [int(x) for x in torch.randint(3, 21, (Nf,), generator=gf)]
    mask_f = torch.zeros(Nf, 20)
    for r_, l_ in enumerate(rlf):
        mask_f[r_, :l_] = 1.0
    ro_f = A.Rollout(prompt_ids=torch.randint(2, 512, (Nf, 12), generator=gf, dtype=torch.int32).to(dev), prompt_lens=plf,
                     resp_ids=torch.randint(2, 512, (Nf, 20), generator=gf, dtype=torch.int32).to(dev), resp_lens=rlf,
                     old_logp=(-torch.rand(Nf, 20, generator=gf) * 3 * mask_f).to(dev), mask=mask_f.to(dev))
    ro_f.adv = (torch.randn(Nf, 20, generator=gf) * mask_f).to(dev)
    ro_f.returns = (torch.randn(Nf, 20, generator=gf) * mask_f).to(dev)
    falgo = A.AlgoConfig(kl_coef=0.0, micro_tokens=64, head_chunk=64)
    n_mb = len(A._micro(ro_f, falgo))
    want_a = A.policy_train_step(whole_a, ro_f, falgo)
    want_c = A.critic_train_step(whole_c, ro_f, falgo)
    sched = uniform_schedule(world, {"actor": n_mb, "critic": n_mb})
    spec = {m.name: m for m in sched.models}
    st_a = LlamaModel(fcfg_a, dev, trainable=True, seed=1, stage=(logical_stage(spec["actor"], rank), world))
    st_c = LlamaModel(fcfg_c, dev, trainable=True, seed=1, stage=(logical_stage(spec["critic"], rank), world))
    for stg, whole_m in ((st_a, whole_a), (st_c, whole_c)):
        for name in stg.layout.entries:
            stg.p[name].copy_(whole_m.p[name])
    fx = FusedPipelineExecutor({"actor": st_a, "critic": st_c}, sched)
    got_f = A.fused_actor_critic_train_step(st_a, st_c, ro_f, falgo, fx)
    torch.cuda.synchronize()
    K.check_status()
    f_ok = [n_mb >= world, abs(float(got_f["loss"]) - float(want_a["loss"])) < 2e-3 * max(1.0, abs(float(want_a["loss"]))),
            abs(float(got_f["value_loss"]) - float(want_c["value_loss"])) < 2e-3 * max(1.0, abs(float(want_c["value_loss"])))]
    for stg, whole_m in ((st_a, whole_a), (st_c, whole_c)):
        for name in stg.layout.entries:
            a_, b_ = stg.gp[name].float(), whole_m.gp[name].float()
            f_ok.append(bool(((a_ - b_).norm() <= 3e-2 * b_.norm() + 1e-6).item()))
    report["fused_actor_critic_pipeline_ok"] = all(f_ok)
    dist.barrier()

    _progress(rank, "10")
    # 10 disaggregated GRPO with staleness 1: the first half of the ranks generate, the second half train; weights and
    #    rollouts cross through versioned peer-memory channels only
    from ..engine.async_rl import AsyncGRPO
    half = world // 2
    acfg = LlamaConfig.tiny(n_layers=2, vocab=512)
    eng = AsyncGRPO(acfg, gen_ranks=list(range(half)), train_ranks=list(range(half, world)), prompts_per_step=2 * half,
                    samples_per_prompt=4, max_new=16, prompt_len=8, tau=1, algo=A.AlgoConfig(kl_coef=0.04, micro_tokens=256, head_chunk=128),
                    lr=1e-3, gen_slots=8, kv_budget_bytes=5e8, seed=3, eos_id=1, device=dev, wait_timeout_s=120.0)
    ga = torch.Generator().manual_seed(17)
    seen = []
    for it in range(3):
        pr = torch.randint(2, acfg.vocab, (2 * half, 8), generator=ga, dtype=torch.int32)
        rw = torch.randn(2 * half * 4, generator=ga)
        seen.append(eng.step(pr, rw))
    if eng.is_gen:
        async_ok = [m["weight_version"] for m in seen] == [0.0, 0.0, 1.0] and eng.weights.ready(3, 60.0)
        final = eng.weights.slot_weights(3).float().sum().reshape(1).double() if async_ok else torch.zeros(1, dtype=torch.float64, device=dev)
    else:
        async_ok = [m["published_version"] for m in seen] == [1.0, 2.0, 3.0] and all(m["loss"] == m["loss"] for m in seen)
        final = eng.actor.w[: eng.actor.layout.total].float().sum().reshape(1).double()
    torch.cuda.synchronize()
    lo, hi = final.clone(), final.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    report["async_staleness_ok"] = bool(async_ok) and bool((lo == hi).item())
    guards_intact("asynchronous GRPO channels")
    eng.close()
    report["symmetric_guards_intact"] = all(guards)

    flags = torch.tensor([float(all(v for k, v in report.items() if k not in ("world", "pipeline_p2p_calls")))], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    report["ok"] = bool(flags.item() == 1.0)
    if rank == 0:
        print(json.dumps(report))
    else:
        bad = {k: v for k, v in report.items() if v is False}
        if bad:
            print(json.dumps({"rank": rank, "failed": bad}), file=sys.stderr)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
