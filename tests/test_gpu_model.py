"""End-to-end numerics of the native model path against plain PyTorch fp32 on the same weights."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from rpeg_b200.engine import algorithms as A  # noqa: E402
from rpeg_b200.engine.generation import Generator  # noqa: E402
from rpeg_b200.engine.optimizer import AdamW  # noqa: E402
from rpeg_b200.engine.trainers import DPOTrainer, GRPOTrainer, PPOTrainer  # noqa: E402
from rpeg_b200.models.llama import LlamaConfig, LlamaModel  # noqa: E402
from rpeg_b200.ops import kernels as K  # noqa: E402


def _ref_forward(model: LlamaModel, params, tokens, lens):
    """fp32 PyTorch restatement of the decoder on packed sequences (one at a time)."""
    cfg = model.cfg
    outs = []
    off = 0
    for L in lens:
        ids = tokens[off:off + L].long()
        h = params["embed"][ids]
        pos = torch.arange(L, device=h.device)
        cos, sin = model.cos_t[pos][:, None, :], model.sin_t[pos][:, None, :]

        def rope(x):
            x1, x2 = x[..., :64], x[..., 64:]
            return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

        def norm(x, w):
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w

        for i in range(cfg.n_layers):
            x = norm(h, params[f"l{i}.attn_norm"])
            qkv = x @ params[f"l{i}.wqkv"].t()
            q = qkv[:, :cfg.q_width].view(L, cfg.n_heads, 128)
            k = qkv[:, cfg.q_width:cfg.q_width + cfg.kv_width].view(L, cfg.n_kv_heads, 128)
            if cfg.qk_norm:
                q, k = norm(q, params[f"l{i}.q_norm"]), norm(k, params[f"l{i}.k_norm"])
            G = cfg.n_heads // cfg.n_kv_heads
            q, k = rope(q), rope(k).repeat_interleave(G, 1)
            v = qkv[:, cfg.q_width + cfg.kv_width:].view(L, cfg.n_kv_heads, 128).repeat_interleave(G, 1)
            s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(128)
            s = s.masked_fill(torch.triu(torch.ones(L, L, dtype=torch.bool, device=h.device), 1), float("-inf"))
            a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(L, cfg.q_width)
            h = h + a @ params[f"l{i}.wo"].t()
            x2 = norm(h, params[f"l{i}.mlp_norm"])
            gu = x2 @ params[f"l{i}.w_gate_up"].t()
            h = h + (torch.nn.functional.silu(gu[:, :cfg.d_ff]) * gu[:, cfg.d_ff:]) @ params[f"l{i}.w_down"].t()
        outs.append(norm(h, params["final_norm"]))
        off += L
    return torch.cat(outs)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("recompute,variant", [("full", "llama"), ("none", "llama"), ("full", "qwen3"), ("none", "qwen3"),
                                               ("keep the last layer", "llama"), ("keep the last layer", "qwen3")])
def test_forward_backward_matches_pytorch(cuda_device, recompute, variant):
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny() if variant == "llama" else LlamaConfig.tiny(
        d_model=512, n_heads=4, n_kv_heads=2, qk_norm=True, tie_embeddings=True, rope_scaling_factor=8.0, rms_eps=1e-6, family="qwen3")
    model = LlamaModel(cfg, cuda_device, trainable=True, recompute="full" if recompute.startswith("keep") else recompute, seed=1)
    if recompute.startswith("keep"):
        model.keep_layers = 1          # layer 1 keeps its activations, layer 0 is recomputed from its input
    lens = [37, 130, 200]
    T = sum(lens)
    tokens = torch.randint(0, cfg.vocab, (T,), device=cuda_device, dtype=torch.int32)
    pos = torch.cat([torch.arange(l) for l in lens]).to(cuda_device, torch.int32)
    cu = torch.tensor([0, 37, 167, 367], device=cuda_device, dtype=torch.int32)
    targets = torch.randint(0, cfg.vocab, (T,), device=cuda_device, dtype=torch.int32)
    coef = torch.randn(T, device=cuda_device) / T

    xf, ctx = model.forward(tokens, pos, cu, max(lens), keep=True)
    logp, d_xf = model.lm_head_fwd_bwd(xf, targets, lambda s, e, lp: coef[s:e], chunk=128)
    model.backward(ctx, d_xf)
    K.check_status()

    params = {n: v.float().clone().requires_grad_(True) for n, v in model.p.items() if not (cfg.tie_embeddings and n == "lm_head")}
    if cfg.tie_embeddings:
        params["lm_head"] = params["embed"]
        for i in range(cfg.n_layers):            # make the norm weights non-trivial
            assert f"l{i}.q_norm" in params
    xf_ref = _ref_forward(model, params, tokens, lens)
    lp_ref = torch.log_softmax(xf_ref @ params["lm_head"].t(), -1).gather(1, targets.long()[:, None])[:, 0]
    (lp_ref * coef).sum().backward()

    assert _rel(xf, xf_ref) < 2e-2
    assert torch.allclose(logp, lp_ref, atol=5e-2)
    names = ["l1.w_down", "l1.w_gate_up", "l1.wo", "l1.wqkv", "l0.wqkv", "l0.mlp_norm", "final_norm", "embed"]
    names += ["l0.q_norm", "l1.k_norm"] if cfg.qk_norm else []
    names += [] if cfg.tie_embeddings else ["lm_head"]
    for name in names:
        assert _rel(model.gp[name], params[name].grad) < 6e-2, name


def test_generation_matches_packed_forward(cuda_device):
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(n_layers=3)
    model = LlamaModel(cfg, cuda_device, seed=3)
    gen = Generator(model, max_slots=8, max_seq_len=256, kv_budget_bytes=2e9, eos_id=1, sync_interval=4)
    N, S, T = 13, 40, 70     # more rows than slots: exercises admission, retirement and compaction
    prompts = torch.randint(2, cfg.vocab, (N, S), device=cuda_device, dtype=torch.int32)
    forced = [5, 70, 1, 33, 70, 12, 64, 65, 2, 70, 40, 7, 19]
    res = gen.generate(prompts, T, temperature=1.0, seed=7, forced_lens=forced)
    K.check_status()
    lens = res.lengths.tolist()
    assert all(l <= f for l, f in zip(lens, forced))          # natural EOS may end a row earlier
    for i, l in enumerate(lens):
        assert res.tokens[i, l - 1].item() == 1 or l == T
    ro = A.Rollout(prompts, [S] * N, res.tokens, lens, res.logprobs, res.response_mask())
    lp = A.sequence_logprobs(model, ro, A.AlgoConfig(micro_tokens=512, head_chunk=64))
    mask = res.response_mask().bool()
    assert torch.allclose(lp[mask], res.logprobs[mask], atol=6e-2)
    # eager (no graph) decode gives the same tokens when sampling greedily
    a = Generator(model, max_slots=8, max_seq_len=256, kv_budget_bytes=2e9, eos_id=1, use_graphs=False).generate(
        prompts[:4], 16, greedy=True)
    b = gen.generate(prompts[:4], 16, greedy=True)
    assert torch.equal(a.tokens, b.tokens)


def test_adamw_updates_model(cuda_device):
    cfg = LlamaConfig.tiny()
    model = LlamaModel(cfg, cuda_device, trainable=True, seed=0)
    opt = AdamW(model, lr=1e-3, max_grad_norm=1.0)
    before = model.w.clone()
    model.g.normal_()
    opt.step()
    assert not torch.equal(before, model.w)
    assert abs(opt.grad_norm().item() - model.g.norm().item()) / model.g.norm().item() < 1e-3
    assert torch.equal(model.w, opt.master.bfloat16())


def test_grpo_ppo_dpo_steps_run_and_learn(cuda_device):
    cfg = LlamaConfig.tiny()
    algo = A.AlgoConfig(kl_coef=0.05, micro_tokens=1024, head_chunk=256)
    grpo = GRPOTrainer(cfg, device=cuda_device, samples_per_prompt=4, max_new=24, prompt_len=16, algo=algo, lr=1e-4,
                       gen_slots=8, kv_budget_bytes=1e9, eos_id=1, sync_interval=4)
    prompts = torch.randint(2, cfg.vocab, (4, 16), dtype=torch.int32).pin_memory()
    rewards = torch.randn(16).pin_memory()
    w0 = grpo.actor.w.clone()
    out = grpo.step(prompts, rewards, forced_lens=torch.randint(1, 25, (16,)))
    assert math.isfinite(out["loss"]) and out["samples"] == 16 and out["gen_tokens"] > 0
    assert not torch.equal(w0, grpo.actor.w) and grpo.weight_version == 1
    out2 = grpo.step(prompts, rewards)
    assert math.isfinite(out2["loss"]) and out2["grad_norm"] > 0

    ppo = PPOTrainer(cfg, device=cuda_device, max_new=16, prompt_len=16, algo=A.AlgoConfig(micro_tokens=512, head_chunk=128),
                     gen_slots=8, kv_budget_bytes=1e9, eos_id=1, lr_actor=1e-4, lr_critic=1e-4)
    o = ppo.step(prompts)
    assert math.isfinite(o["loss"]) and math.isfinite(o["value_loss"])
    ppo_shared = PPOTrainer(cfg, device=cuda_device, max_new=16, prompt_len=16, share_actor_critic=True,
                            algo=A.AlgoConfig(micro_tokens=512, head_chunk=128), gen_slots=8, kv_budget_bytes=1e9, eos_id=1)
    o = ppo_shared.step(prompts)
    assert math.isfinite(o["loss"]) and math.isfinite(o["value_loss"])

    dpo = DPOTrainer(cfg, device=cuda_device, algo=A.AlgoConfig(beta=0.1, micro_tokens=512, head_chunk=128), lr=1e-4)
    P, S, T = 6, 12, 20
    pr = torch.randint(2, cfg.vocab, (P, S), dtype=torch.int32).repeat_interleave(2, 0).pin_memory()
    rs = torch.randint(2, cfg.vocab, (2 * P, T), dtype=torch.int32).pin_memory()
    first = dpo.step(pr, rs)
    assert abs(first["loss"] - math.log(2.0)) < 1e-3          # policy == reference at step 0
    for _ in range(5):
        last = dpo.step(pr, rs)
    assert last["loss"] < first["loss"]                        # the pair loss goes down on a fixed batch
    K.check_status()


@pytest.mark.gpu
def test_generation_with_page_preemption_matches_roomy_pool(cuda_device):
    """A pool too small for all live rows forces preemptions; greedy decoding must still give the
    tokens a roomy pool gives, and every page must come back."""
    cfg = LlamaConfig.tiny(n_layers=2)
    model = LlamaModel(cfg, cuda_device, seed=5)
    N, S, T = 10, 60, 200
    prompts = torch.randint(2, cfg.vocab, (N, S), device=cuda_device, dtype=torch.int32)
    forced = [200, 150, 200, 30, 200, 180, 90, 200, 200, 120]
    page_bytes = 2 * cfg.n_layers * cfg.n_kv_heads * K.KV_PAGE * cfg.head_dim * 2
    roomy = Generator(model, max_slots=8, max_seq_len=S + T, kv_budget_bytes=1e9, eos_id=1, sync_interval=4)
    tight = Generator(model, max_slots=8, max_seq_len=S + T, kv_budget_bytes=15.5 * page_bytes, eos_id=1, sync_interval=4)
    a = roomy.generate(prompts, T, greedy=True, forced_lens=forced)
    b = tight.generate(prompts, T, greedy=True, forced_lens=forced)
    K.check_status()
    assert a.counters["kv_preemptions"] == 0 and b.counters["kv_preemptions"] > 0
    assert torch.equal(a.lengths, b.lengths)
    # batch composition changes the GEMM split, so a near-tie may flip a greedy choice: most rows agree exactly ...
    same = sum(int(torch.equal(a.tokens[i], b.tokens[i])) for i in range(N))
    assert same >= N - 2, f"only {same} of {N} rows identical"
    # ... and every row of the preempted run is consistent with a packed forward over its own tokens
    lens = b.lengths.tolist()
    ro = A.Rollout(prompts, [S] * N, b.tokens, lens, b.logprobs, b.response_mask())
    lp = A.sequence_logprobs(model, ro, A.AlgoConfig(micro_tokens=1024, head_chunk=64))
    mask = b.response_mask().bool()
    assert torch.allclose(lp[mask], b.logprobs[mask], atol=6e-2)
    for r in (a, b):
        assert r.counters["kv_pages_taken"] == r.counters["kv_pages_returned"]
    assert tight.pool.available() == tight.pool.num_pages - 1


@pytest.mark.parametrize("S", [128, 150])
def test_generation_with_shared_prompt_pages(cuda_device, S):
    """K samples per prompt with the prompt's KV pages shared by the group: one prefill per prompt, fewer pages, and
    every sampled row consistent with a packed forward over its own tokens. Prompt lengths: a whole number of pages
    and a ragged tail (the tail page is copied per row). A tight pool forces preemptions and late admissions that
    alias prompts prefilled earlier; every page must come back."""
    cfg = LlamaConfig.tiny(n_layers=2)
    model = LlamaModel(cfg, cuda_device, seed=9)
    P, Kq, T = 5, 4, 90
    uniq = torch.randint(2, cfg.vocab, (P, S), device=cuda_device, dtype=torch.int32)
    prompts = uniq.repeat_interleave(Kq, dim=0).contiguous()
    N = P * Kq
    forced = [(17 * i) % T + 1 for i in range(N)]
    page_bytes = 2 * cfg.n_layers * cfg.n_kv_heads * K.KV_PAGE * cfg.head_dim * 2
    plain = Generator(model, max_slots=8, max_seq_len=S + T, kv_budget_bytes=1e9, eos_id=1, sync_interval=4)
    shared = Generator(model, max_slots=8, max_seq_len=S + T, kv_budget_bytes=1e9, eos_id=1, sync_interval=4)
    tight = Generator(model, max_slots=8, max_seq_len=S + T, kv_budget_bytes=14.5 * page_bytes, eos_id=1, sync_interval=4,
                      group_attention=True)
    tight.group_min_batch = 0          # the group kernel at every batch size, not only while many rows are live
    a = plain.generate(prompts, T, seed=11, forced_lens=forced)
    b = shared.generate(prompts, T, seed=11, forced_lens=forced, group_size=Kq)
    c = tight.generate(prompts, T, seed=11, forced_lens=forced, group_size=Kq)
    K.check_status()
    assert a.counters["prompts_prefilled"] == N and b.counters["prompts_prefilled"] == P and c.counters["prompts_prefilled"] == P
    assert b.counters["shared_prompt_pages"] == P * (S // K.KV_PAGE)
    assert b.counters["kv_pages_taken"] < a.counters["kv_pages_taken"]
    assert c.counters["kv_preemptions"] > 0
    for res, g in ((a, plain), (b, shared), (c, tight)):
        assert res.counters["kv_pages_taken"] == res.counters["kv_pages_returned"]
        assert g.pool.available() == g.pool.num_pages - 1
        lens = res.lengths.tolist()
        assert all(1 <= l <= f for l, f in zip(lens, forced))
        ro = A.Rollout(prompts, [S] * N, res.tokens, lens, res.logprobs, res.response_mask())
        lp = A.sequence_logprobs(model, ro, A.AlgoConfig(micro_tokens=1024, head_chunk=64))
        mask = res.response_mask().bool()
        assert torch.allclose(lp[mask], res.logprobs[mask], atol=6e-2)
    # greedy decoding: sharing must not change what a row generates (up to near-tie flips from the batch composition)
    ga = plain.generate(prompts, 24, greedy=True)
    gb = shared.generate(prompts, 24, greedy=True, group_size=Kq)
    same = sum(int(torch.equal(ga.tokens[i], gb.tokens[i])) for i in range(N))
    assert same >= N - 2, f"only {same} of {N} rows identical"
    # the group attention kernel (shared keys scored once per group) must agree with the row-by-row kernel
    grouped = Generator(model, max_slots=32, max_seq_len=S + T, kv_budget_bytes=1e9, eos_id=1, sync_interval=4, group_attention=True)
    grouped.group_min_batch = 0
    gc = grouped.generate(prompts, 24, greedy=True, group_size=Kq)
    K.check_status()
    same = sum(int(torch.equal(ga.tokens[i], gc.tokens[i])) for i in range(N))
    assert same >= N - 2, f"group attention: only {same} of {N} rows identical"
    gd = grouped.generate(prompts, T, seed=11, forced_lens=forced, group_size=Kq)
    lens = gd.lengths.tolist()
    ro = A.Rollout(prompts, [S] * N, gd.tokens, lens, gd.logprobs, gd.response_mask())
    lp = A.sequence_logprobs(model, ro, A.AlgoConfig(micro_tokens=1024, head_chunk=64))
    mask = gd.response_mask().bool()
    assert torch.allclose(lp[mask], gd.logprobs[mask], atol=6e-2)


def test_generation_with_top_k_stays_inside_the_top_k(cuda_device):
    """``top_k = 1`` through the whole generator (prefill sampling, graph decode steps) equals greedy decoding, and the
    recorded log-probs are those of the full softmax."""
    cfg = LlamaConfig.tiny(n_layers=2)
    model = LlamaModel(cfg, cuda_device, seed=4)
    gen = Generator(model, max_slots=8, max_seq_len=128, kv_budget_bytes=5e8, eos_id=1, sync_interval=4)
    prompts = torch.randint(2, cfg.vocab, (6, 20), device=cuda_device, dtype=torch.int32)
    a = gen.generate(prompts, 24, greedy=True)
    b = gen.generate(prompts, 24, temperature=1.0, seed=3, top_k=1)
    K.check_status()
    same = sum(int(torch.equal(a.tokens[i], b.tokens[i])) for i in range(6))
    assert same >= 5, f"only {same} of 6 rows identical"          # a bf16 tie may flip one choice
    lens = b.lengths.tolist()
    ro = A.Rollout(prompts, [20] * 6, b.tokens, lens, b.logprobs, b.response_mask())
    lp = A.sequence_logprobs(model, ro, A.AlgoConfig(micro_tokens=512, head_chunk=64))
    mask = b.response_mask().bool()
    assert torch.allclose(lp[mask], b.logprobs[mask], atol=6e-2)
    c = gen.generate(prompts, 24, temperature=1.0, seed=3, top_p=0.3)
    K.check_status()
    assert int(c.lengths.min()) >= 1
