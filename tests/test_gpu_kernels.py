"""Numerics of every single-GPU sm_100a kernel against a plain PyTorch fp32 reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from rpeg_b200.ops import kernels as K  # noqa: E402


def _rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_clean(cuda_device):
    torch.manual_seed(0)
    yield
    K.check_status()


GEMM_SHAPES = [
    (128, 256, 64), (256, 512, 256), (300, 264, 200), (1024, 4096, 4096), (4096, 11008, 4096),
    (32, 4096, 4096), (8, 32000, 4096), (64, 12288, 4096), (5, 40, 72),
]


@pytest.mark.parametrize("M,N,K_", GEMM_SHAPES)
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(cuda_device, M, N, K_, trans_a, trans_b):
    if trans_a and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0")
    a = torch.randn((K_, M) if trans_a else (M, K_), device=cuda_device).bfloat16()
    b = torch.randn((K_, N) if trans_b else (N, K_), device=cuda_device).bfloat16()
    ref = (a.float().t() if trans_a else a.float()) @ (b.float() if trans_b else b.float().t())
    out = K.gemm(a, b, trans_a=trans_a, trans_b=trans_b)
    assert _rel_err(out, ref) < 1e-2
    out32 = K.gemm(a, b, trans_a=trans_a, trans_b=trans_b, out_dtype=torch.float32)
    assert _rel_err(out32, ref) < 2e-3


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_gemm_tile_widths_and_accumulate(cuda_device, bn):
    M, N, K_ = 384, 768, 520
    a = torch.randn(M, K_, device=cuda_device).bfloat16()
    b = torch.randn(N, K_, device=cuda_device).bfloat16()
    ref = a.float() @ b.float().t()
    assert _rel_err(K.gemm(a, b, bn=bn), ref) < 1e-2
    acc = torch.ones(M, N, device=cuda_device)
    K.gemm(a, b, out=acc, accumulate=True, bn=bn)
    assert _rel_err(acc, ref + 1.0) < 2e-3


def test_gemm_strided_rows(cuda_device):
    big = torch.randn(256, 3 * 512, device=cuda_device).bfloat16()
    a = big[:, 512:1024]
    w = torch.randn(384, 512, device=cuda_device).bfloat16()
    assert _rel_err(K.gemm(a, w), a.float() @ w.float().t()) < 1e-2


@pytest.mark.parametrize("T,d", [(7, 256), (1000, 4096), (33, 5120)])
def test_rmsnorm_fwd_bwd(cuda_device, T, d):
    x = torch.randn(T, d, device=cuda_device).bfloat16()
    res = torch.randn(T, d, device=cuda_device).bfloat16()
    w = (1 + 0.1 * torch.randn(d, device=cuda_device)).bfloat16()
    eps = 1e-5
    y, rstd, h = K.rmsnorm_fwd(x, w, eps, residual=res, want_sum=True)
    h_ref = (x.float() + res.float()).bfloat16()
    assert torch.equal(h, h_ref)
    hf = h_ref.float()
    rs_ref = torch.rsqrt(hf.pow(2).mean(-1) + eps)
    assert _rel_err(rstd, rs_ref) < 1e-4
    assert _rel_err(y, hf * rs_ref[:, None] * w.float()) < 5e-3
    # backward against autograd on fp32
    dy = torch.randn(T, d, device=cuda_device).bfloat16()
    dres = torch.randn(T, d, device=cuda_device).bfloat16()
    hx = hf.clone().requires_grad_(True)
    wf = w.float().clone().requires_grad_(True)
    yy = hx * torch.rsqrt(hx.pow(2).mean(-1, keepdim=True) + eps) * wf
    yy.backward(dy.float())
    dw = torch.zeros(d, device=cuda_device)
    dx = K.rmsnorm_bwd(dy, h_ref, w, rstd, dw, dres_in=dres)
    assert _rel_err(dx, hx.grad + dres.float()) < 1e-2
    assert _rel_err(dw, wf.grad) < 1e-2


def test_rope_roundtrip_and_reference(cuda_device):
    T, H, hd = 300, 4, 128
    buf = torch.randn(T, 3 * H * hd, device=cuda_device).bfloat16()
    orig = buf.clone()
    pos = torch.randint(0, 2048, (T,), device=cuda_device, dtype=torch.int32)
    cos_t, sin_t = K.rope_tables(2048, hd, 10000.0, cuda_device)
    K.rope_(buf, pos, cos_t, sin_t, H * hd, H, hd)  # rotate the K block only
    k = orig[:, H * hd:2 * H * hd].float().view(T, H, hd)
    c = cos_t[pos.long()][:, None, :]
    s = sin_t[pos.long()][:, None, :]
    k1, k2 = k[..., :hd // 2], k[..., hd // 2:]
    ref = torch.cat([k1 * c - k2 * s, k2 * c + k1 * s], -1).view(T, H * hd)
    assert _rel_err(buf[:, H * hd:2 * H * hd], ref) < 5e-3
    assert torch.equal(buf[:, :H * hd], orig[:, :H * hd]) and torch.equal(buf[:, 2 * H * hd:], orig[:, 2 * H * hd:])
    K.rope_(buf, pos, cos_t, sin_t, H * hd, H, hd, backward=True)
    assert _rel_err(buf, orig) < 1e-2


def test_swiglu(cuda_device):
    T, f = 257, 1408
    gu = torch.randn(T, 2 * f, device=cuda_device).bfloat16()
    dout = torch.randn(T, f, device=cuda_device).bfloat16()
    g = gu[:, :f].float().clone().requires_grad_(True)
    u = gu[:, f:].float().clone().requires_grad_(True)
    ref = torch.nn.functional.silu(g) * u
    ref.backward(dout.float())
    assert _rel_err(K.swiglu_fwd(gu), ref) < 5e-3
    dgu = K.swiglu_bwd(gu, dout)
    assert _rel_err(dgu[:, :f], g.grad) < 1e-2 and _rel_err(dgu[:, f:], u.grad) < 1e-2


def test_embedding(cuda_device):
    V, d, T = 1000, 256, 513
    table = torch.randn(V, d, device=cuda_device).bfloat16()
    ids = torch.randint(0, V, (T,), device=cuda_device, dtype=torch.int32)
    assert torch.equal(K.embed_fwd(ids, table), table[ids.long()])
    dout = torch.randn(T, d, device=cuda_device).bfloat16()
    dt = torch.zeros(V, d, device=cuda_device)
    K.embed_bwd(ids, dout, dt)
    ref = torch.zeros(V, d, device=cuda_device).index_add_(0, ids.long(), dout.float())
    assert _rel_err(dt, ref) < 1e-5


@pytest.mark.parametrize("V", [32000, 1003])
def test_token_logprob_fwd_bwd(cuda_device, V):
    T = 77
    ld = (V + 7) // 8 * 8
    store = (3 * torch.randn(T, ld, device=cuda_device)).bfloat16()
    logits = store[:, :V]
    tgt = torch.randint(0, V, (T,), device=cuda_device, dtype=torch.int32)
    lf = logits.float().clone().requires_grad_(True)
    ref = torch.log_softmax(lf, -1).gather(1, tgt.long()[:, None])[:, 0]
    logp, lse = K.token_logprob_fwd(logits, tgt)
    assert torch.allclose(logp, ref, atol=2e-3, rtol=1e-3)
    coef = torch.randn(T, device=cuda_device)
    ref.backward(coef)
    K.token_logprob_bwd_(logits, tgt, lse, coef)
    assert _rel_err(logits, lf.grad) < 1e-2


def test_policy_loss(cuda_device):
    n = 5000
    lp = -torch.rand(n, device=cuda_device) * 3
    old = lp + 0.3 * torch.randn(n, device=cuda_device)
    refp = lp + 0.1 * torch.randn(n, device=cuda_device)
    adv = torch.randn(n, device=cuda_device)
    mask = (torch.rand(n, device=cuda_device) > 0.3).float()
    eps, klc = 0.2, 0.05
    denom = mask.sum().item()
    x = lp.clone().requires_grad_(True)
    ratio = torch.exp(x - old)
    pg = -torch.minimum(ratio * adv, torch.clamp(ratio, 1 - eps, 1 + eps) * adv)
    loss = ((pg + klc * (x - refp)) * mask).sum() / denom
    loss.backward()
    coef, acc = K.policy_loss(lp, old, refp, adv, mask, eps, klc, 1.0 / denom)
    assert abs(acc[0].item() - loss.item()) < 1e-4
    assert torch.allclose(coef, x.grad, atol=1e-6, rtol=1e-4)


def test_dpo_loss(cuda_device):
    P, T = 16, 40
    beta = 0.1
    lp = -torch.rand(2 * P, T, device=cuda_device)
    mask = (torch.rand(2 * P, T, device=cuda_device) > 0.4).float()
    ref_seq = -torch.rand(2 * P, device=cuda_device) * 10
    x = lp.clone().requires_grad_(True)
    seq = (x * mask).sum(-1)
    z = beta * ((seq[0::2] - seq[1::2]) - (ref_seq[0::2] - ref_seq[1::2]))
    loss = -torch.nn.functional.logsigmoid(z).mean()
    loss.backward()
    pi_seq = K.masked_rowsum(lp, mask)
    assert torch.allclose(pi_seq, seq.detach(), atol=1e-4)
    seq_coef, acc = K.dpo_loss(pi_seq, ref_seq, beta)
    coef = K.expand_seq_coef(seq_coef, mask)
    assert abs(acc[0].item() - loss.item()) < 1e-5
    assert torch.allclose(coef, x.grad, atol=1e-6, rtol=1e-4)


def test_value_loss_and_gae(cuda_device):
    B, T = 9, 50
    lens = torch.randint(1, T + 1, (B,), device=cuda_device)
    mask = (torch.arange(T, device=cuda_device)[None, :] < lens[:, None]).float()
    v = torch.randn(B, T, device=cuda_device)
    old = -torch.rand(B, T, device=cuda_device)
    refp = -torch.rand(B, T, device=cuda_device)
    scores = torch.randn(B, device=cuda_device)
    beta, gamma, lam = 0.1, 0.99, 0.95
    adv, ret = K.gae(old, refp, v, mask, scores, beta, gamma, lam, whiten=False)
    r = -beta * (old - refp) * mask
    r[torch.arange(B), lens - 1] += scores
    a_ref = torch.zeros(B, T, device=cuda_device)
    a_next = torch.zeros(B, device=cuda_device)
    for t in reversed(range(T)):
        v_next = v[:, t + 1] * mask[:, t + 1] if t + 1 < T else torch.zeros(B, device=cuda_device)
        m_next = mask[:, t + 1] if t + 1 < T else torch.zeros(B, device=cuda_device)
        delta = r[:, t] + gamma * v_next - v[:, t]
        a_next = delta + gamma * lam * m_next * a_next
        a_ref[:, t] = a_next * mask[:, t]
    assert torch.allclose(adv, a_ref, atol=1e-4, rtol=1e-4)
    assert torch.allclose(ret, (a_ref + v) * mask, atol=1e-4, rtol=1e-4)
    adv_w, _ = K.gae(old, refp, v, mask, scores, beta, gamma, lam, whiten=True)
    n = mask.sum()
    mean = (a_ref * mask).sum() / n
    var = (((a_ref - mean) * mask) ** 2).sum() / n
    assert torch.allclose(adv_w, (a_ref - mean) * torch.rsqrt(var + 1e-6) * mask, atol=1e-3, rtol=1e-3)
    dv, acc = K.value_loss(v, ret, mask, 1.0 / n.item())
    assert abs(acc[0].item() - (((v - ret) * mask) ** 2).sum().item() / n.item()) < 1e-4
    assert torch.allclose(dv, 2 * (v - ret) * mask / n, atol=1e-6)


def test_group_advantage(cuda_device):
    r = torch.randn(8 * 4, device=cuda_device)
    out = K.group_advantage(r, 4)
    g = r.view(8, 4)
    ref = (g - g.mean(1, keepdim=True)) / g.std(1, unbiased=False, keepdim=True).clamp_min(1e-6)
    assert torch.allclose(out.view(8, 4), ref, atol=1e-5)


def test_sampler(cuda_device):
    B, V = 64, 1000
    logits = (2 * torch.randn(B, V, device=cuda_device)).bfloat16()
    tok, lp = K.sample(logits, 1.0, True, 1)
    assert torch.equal(tok.long(), logits.float().argmax(-1))
    ref_lp = torch.log_softmax(logits.float(), -1)
    assert torch.allclose(lp, ref_lp.gather(1, tok.long()[:, None])[:, 0], atol=2e-3)
    # sampled frequencies follow the softmax (one shared distribution, many rows)
    row = torch.tensor([2.0, 1.0, 0.0, -1.0] + [-20.0] * 12, device=cuda_device).bfloat16()
    many = row[None, :].expand(20000, 16).contiguous()
    tok, _ = K.sample(many, 1.0, False, 1234)
    freq = torch.bincount(tok.long(), minlength=16).float() / 20000
    assert torch.allclose(freq, torch.softmax(row.float(), -1), atol=0.02)
    forced = torch.full((B,), -1, device=cuda_device, dtype=torch.int32)
    forced[3] = 7
    tok, lp = K.sample(logits, 1.0, False, 5, forced=forced)
    assert tok[3].item() == 7 and abs(lp[3].item() - ref_lp[3, 7].item()) < 2e-3
    # a vocabulary-sized row (16-byte loads), a row length that is no multiple of 8 and rows that start off a 16-byte
    # boundary (scalar loads): the same argmax and log-prob on both paths
    for rows, width in ((8, 32000), (5, 1003), (3, 1001)):
        wide = (3 * torch.randn(rows, width, device=cuda_device)).bfloat16()
        tok, lp = K.sample(wide, 0.7, True, 9)
        assert torch.equal(tok.long(), wide.float().argmax(-1))
        want = torch.log_softmax(wide.float() / 0.7, -1).gather(1, tok.long()[:, None])[:, 0]
        assert torch.allclose(lp, want, atol=3e-3)
        drawn, _ = K.sample(wide, 0.7, False, 77)
        again, _ = K.sample(wide, 0.7, False, 77)
        assert torch.equal(drawn, again) and int(drawn.max()) < width


def test_scalar_head(cuda_device):
    T, d = 300, 512
    h = torch.randn(T, d, device=cuda_device).bfloat16()
    w = (0.05 * torch.randn(d, device=cuda_device)).bfloat16()
    b = torch.tensor([0.3], device=cuda_device)
    out = K.head_gemv(h, w, b)
    assert torch.allclose(out, h.float() @ w.float() + 0.3, atol=1e-3, rtol=1e-3)
    dout = torch.randn(T, device=cuda_device)
    dw = torch.zeros(d, device=cuda_device)
    db = torch.zeros(1, device=cuda_device)
    dh = K.head_gemv_bwd(h, w, dout, dw, db)
    assert _rel_err(dh, dout[:, None] * w.float()[None, :]) < 5e-3
    assert _rel_err(dw, dout @ h.float()) < 1e-4
    assert abs(db.item() - dout.sum().item()) < 1e-3


def test_adamw_matches_torch(cuda_device):
    n = 4096 * 3
    p = torch.randn(n, device=cuda_device)
    g = torch.randn(n, device=cuda_device)
    ref_p = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    m = torch.zeros(n, device=cuda_device)
    v = torch.zeros(n, device=cuda_device)
    w16 = torch.empty(n, device=cuda_device, dtype=torch.bfloat16)
    for step in range(1, 4):
        ref_p.grad = g.clone()
        opt.step()
        K.adamw_(p, m, v, g, w16, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.01, step=step)
    assert torch.allclose(p, ref_p.detach(), atol=1e-5, rtol=1e-4)
    assert torch.equal(w16, p.bfloat16())
    ss = torch.zeros(1, device=cuda_device)
    K.sumsq(g, ss)
    assert abs(ss.item() - g.pow(2).sum().item()) / g.pow(2).sum().item() < 1e-4
    # clip coefficient read on the device: max_norm / (norm + 1e-6), capped at 1
    p2, m2, v2 = torch.zeros(n, device=cuda_device), torch.zeros(n, device=cuda_device), torch.zeros(n, device=cuda_device)
    K.adamw_(p2, m2, v2, g, w16, lr=1.0, beta1=0.0, beta2=0.0, eps=1.0, step=1, sumsq=ss, max_norm=1.0)
    gc = g * min(1.0, 1.0 / (g.norm().item() + 1e-6))
    assert torch.allclose(p2, -(gc / (gc.abs() + 1.0)), atol=1e-6)


def _paged_cache(cuda_device, lens, Hkv, hd, num_pages):
    B = len(lens)
    max_pages = (max(lens) + K.KV_PAGE - 1) // K.KV_PAGE
    perm = torch.randperm(num_pages)[: B * max_pages].view(B, max_pages)
    table = perm.to(device=cuda_device, dtype=torch.int32).contiguous()
    kc = torch.zeros(num_pages, Hkv, K.KV_PAGE, hd, device=cuda_device, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    return table, kc, vc


@pytest.mark.parametrize("nsplit", [1, 4])
@pytest.mark.parametrize("H,Hkv", [(8, 8), (8, 2)])
def test_kv_append_and_paged_decode(cuda_device, nsplit, H, Hkv):
    hd = 128
    lens = [1, 63, 64, 65, 300, 517]
    B = len(lens)
    table, kc, vc = _paged_cache(cuda_device, lens, Hkv, hd, 64)
    T = sum(lens)
    ld = (H + 2 * Hkv) * hd
    qkv = torch.randn(T, ld, device=cuda_device).bfloat16()
    seq_id = torch.cat([torch.full((l,), i) for i, l in enumerate(lens)]).to(cuda_device, torch.int32)
    pos = torch.cat([torch.arange(l) for l in lens]).to(cuda_device, torch.int32)
    K.kv_append(qkv, H * hd, (H + Hkv) * hd, seq_id, pos, table, kc, vc, Hkv, hd)
    q = torch.randn(B, H * hd, device=cuda_device).bfloat16()
    seq_lens = torch.tensor(lens, device=cuda_device, dtype=torch.int32)
    out = K.paged_decode_attn(q, 0, kc, vc, table, seq_lens, H, Hkv, hd, 1 / math.sqrt(hd), nsplit=nsplit)
    off = 0
    for i, l in enumerate(lens):
        kk = qkv[off:off + l, H * hd:(H + Hkv) * hd].float().view(l, Hkv, hd)
        vv = qkv[off:off + l, (H + Hkv) * hd:].float().view(l, Hkv, hd)
        kk = kk.repeat_interleave(H // Hkv, 1)
        vv = vv.repeat_interleave(H // Hkv, 1)
        qq = q[i].float().view(H, hd)
        p = torch.softmax(torch.einsum("hd,lhd->hl", qq, kk) / math.sqrt(hd), -1)
        ref = torch.einsum("hl,lhd->hd", p, vv).reshape(-1)
        assert _rel_err(out[i], ref) < 1e-2, f"sequence {i}"
        off += l


@pytest.mark.parametrize("M,f,Kd", [(300, 512, 256), (128, 1408, 192), (1000, 11008, 128), (5, 128, 64)])
def test_gemm_with_swiglu_epilogue(cuda_device, M, f, Kd):
    """The gated MLP's first linear with silu(gate) * up applied in the GEMM epilogue, against fp32 PyTorch."""
    g = torch.Generator(device="cpu").manual_seed(2)
    x = torch.randn(M, Kd, generator=g).bfloat16().to(cuda_device)
    w = (torch.randn(2 * f, Kd, generator=g) / math.sqrt(Kd)).bfloat16().to(cuda_device)
    out = K.gemm_swiglu(x, w)
    K.check_status()
    gate, up = x.float() @ w[:f].float().t(), x.float() @ w[f:].float().t()
    ref = torch.nn.functional.silu(gate) * up
    assert _rel_err(out, ref) < 1e-2
    two_step = K.swiglu_fwd(K.gemm(x, w))
    assert _rel_err(out, two_step.float()) < 2e-2


@pytest.mark.parametrize("tc", [True, False])
@pytest.mark.parametrize("H,Hkv,shared_pages", [(4, 4, 3), (8, 2, 8), (4, 4, 1)])
def test_paged_decode_attn_with_shared_prompt_groups(cuda_device, tc, H, Hkv, shared_pages):
    """Rows that alias their first KV pages in groups: the group kernel (tensor cores with ``tc``, CUDA cores without)
    scores the shared keys once per group, the per-row kernel the private rest; against fp32 PyTorch over each row's
    own page list. Groups of 8, 5 and 3 rows, one row outside any group, odd and even numbers of shared pages."""
    hd, P = 128, K.KV_PAGE
    g = torch.Generator(device="cpu").manual_seed(4)
    sizes = [8, 5, 3]
    private = [70, 1, 130, 64, 9, 33, 200, 5, 17, 64, 3, 99, 128, 45, 7, 61, 250]      # private keys per row (the last row is ungrouped)
    B = sum(sizes) + 1
    S = shared_pages * P
    max_pages = shared_pages + 5
    n_pages = 1 + len(sizes) * shared_pages + B * 5
    kc = torch.randn(n_pages, Hkv, P, hd, generator=g).bfloat16().to(cuda_device)
    vc = torch.randn(n_pages, Hkv, P, hd, generator=g).bfloat16().to(cuda_device)
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    nxt, row = 1, 0
    group_rows = torch.full((B, 8), -1, dtype=torch.int32)
    group_shared = torch.zeros(B, dtype=torch.int32)
    row_key0 = torch.zeros(B, dtype=torch.int32)
    lens = []
    for gi, n in enumerate(sizes):
        shared = list(range(nxt, nxt + shared_pages))
        nxt += shared_pages
        for j in range(n):
            table[row, :shared_pages] = torch.tensor(shared, dtype=torch.int32)
            own = (private[row] + P - 1) // P
            table[row, shared_pages:shared_pages + own] = torch.arange(nxt, nxt + own, dtype=torch.int32)
            nxt += own
            group_rows[gi, j] = row
            row_key0[row] = S
            lens.append(S + private[row])
            row += 1
        group_shared[gi] = S
    own = (S + private[row] + P - 1) // P                        # the ungrouped row owns all its pages
    table[row, :own] = torch.arange(nxt, nxt + own, dtype=torch.int32)
    lens.append(S + private[row])
    q = torch.randn(B, H * hd, generator=g).bfloat16().to(cuda_device)
    table, seq = table.to(cuda_device), torch.tensor(lens, dtype=torch.int32, device=cuda_device)
    groups = (group_rows.to(cuda_device), group_shared.to(cuda_device), row_key0.to(cuda_device))
    for nsplit in (1, 3):
        out = K.paged_decode_attn(q, 0, kc, vc, table, seq, H, Hkv, hd, 1 / math.sqrt(hd), nsplit=nsplit, groups=groups, group_tc=tc)
        K.check_status()
        for b, l in enumerate(lens):
            pages = table[b, : (l + P - 1) // P].long()
            kk = kc[pages].float().permute(1, 0, 2, 3).reshape(Hkv, -1, hd)[:, :l].repeat_interleave(H // Hkv, 0)
            vv = vc[pages].float().permute(1, 0, 2, 3).reshape(Hkv, -1, hd)[:, :l].repeat_interleave(H // Hkv, 0)
            p = torch.softmax(torch.einsum("hd,hld->hl", q[b].float().view(H, hd), kk) / math.sqrt(hd), -1)
            ref = torch.einsum("hl,hld->hd", p, vv).reshape(-1)
            assert _rel_err(out[b], ref) < 1.5e-2, f"row {b} (nsplit {nsplit})"


@pytest.mark.parametrize("lens", [[128], [5, 130, 257], [1000, 31, 384]])
@pytest.mark.parametrize("H,Hkv", [(4, 4), (4, 2)])
def test_flash_attn_fwd(cuda_device, lens, H, Hkv):
    hd = 128
    T = sum(lens)
    ld = (H + 2 * Hkv) * hd
    qkv = torch.randn(T, ld, device=cuda_device).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=cuda_device, dtype=torch.int32)
    out, lse = K.flash_attn_fwd(qkv, 0, H * hd, (H + Hkv) * hd, cu, max(lens), H, Hkv, hd)
    K.check_status()
    off = 0
    for l in lens:
        q = qkv[off:off + l, :H * hd].float().view(l, H, hd).transpose(0, 1)
        k = qkv[off:off + l, H * hd:(H + Hkv) * hd].float().view(l, Hkv, hd).transpose(0, 1).repeat_interleave(H // Hkv, 0)
        v = qkv[off:off + l, (H + Hkv) * hd:].float().view(l, Hkv, hd).transpose(0, 1).repeat_interleave(H // Hkv, 0)
        s = q @ k.transpose(1, 2) / math.sqrt(hd)
        s = s.masked_fill(torch.triu(torch.ones(l, l, device=cuda_device, dtype=torch.bool), 1), float("-inf"))
        ref = (torch.softmax(s, -1) @ v).transpose(0, 1).reshape(l, H * hd)
        assert _rel_err(out[off:off + l], ref) < 1e-2
        assert torch.allclose(lse[:, off:off + l], torch.logsumexp(s, -1), atol=2e-2, rtol=1e-3)
        off += l


def test_flash_attn_fwd_long_rows_many_heads(cuda_device):
    """32 heads, sequences of 20 to 24 key tiles, several waves of CTAs and repeated launches: the shape of the
    training step, where late K tiles let a P*V product finish before a softmax warp looks at its barrier."""
    hd, H = 128, 32
    lens = [2560, 3072, 2561, 2944]
    T = sum(lens)
    qkv = (torch.randn(T, 3 * H * hd, device=cuda_device) * 0.5).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=cuda_device, dtype=torch.int32)
    out = lse = None
    for _ in range(20):
        out, lse = K.flash_attn_fwd(qkv, 0, H * hd, 2 * H * hd, cu, max(lens), H, H, hd)
    K.check_status()
    off = 0
    for l in lens:
        for h in (0, 13, 31):
            q = qkv[off:off + l, h * hd:(h + 1) * hd].float()
            k = qkv[off:off + l, (H + h) * hd:(H + h + 1) * hd].float()
            v = qkv[off:off + l, (2 * H + h) * hd:(2 * H + h + 1) * hd].float()
            s = q @ k.t() / math.sqrt(hd)
            s = s.masked_fill(torch.triu(torch.ones(l, l, device=cuda_device, dtype=torch.bool), 1), float("-inf"))
            ref = torch.softmax(s, -1) @ v
            assert _rel_err(out[off:off + l, h * hd:(h + 1) * hd], ref) < 1e-2
            assert torch.allclose(lse[h, off:off + l], torch.logsumexp(s, -1), atol=2e-2, rtol=1e-3)
        off += l


@pytest.mark.parametrize("lens", [[128], [5, 130, 257], [1000, 31, 384]])
@pytest.mark.parametrize("H,Hkv", [(4, 4), (4, 2), (8, 2)])
def test_flash_attn_bwd(cuda_device, lens, H, Hkv):
    hd = 128
    G = H // Hkv
    T = sum(lens)
    kc0, vc0, width = H * hd, (H + Hkv) * hd, (H + 2 * Hkv) * hd
    qkv = torch.randn(T, width, device=cuda_device).bfloat16()
    dout = torch.randn(T, H * hd, device=cuda_device).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=cuda_device, dtype=torch.int32)
    out, lse = K.flash_attn_fwd(qkv, 0, kc0, vc0, cu, max(lens), H, Hkv, hd)
    dqkv = K.flash_attn_bwd(qkv, 0, kc0, vc0, out, dout, lse, cu, max(lens), H, Hkv, hd)
    K.check_status()
    x = qkv.float().clone().requires_grad_(True)
    off = 0
    outs = []
    for l in lens:
        q = x[off:off + l, :kc0].view(l, H, hd).transpose(0, 1)
        k = x[off:off + l, kc0:vc0].view(l, Hkv, hd).transpose(0, 1).repeat_interleave(G, 0)
        v = x[off:off + l, vc0:].view(l, Hkv, hd).transpose(0, 1).repeat_interleave(G, 0)
        s = q @ k.transpose(1, 2) / math.sqrt(hd)
        s = s.masked_fill(torch.triu(torch.ones(l, l, device=cuda_device, dtype=torch.bool), 1), float("-inf"))
        outs.append((torch.softmax(s, -1) @ v).transpose(0, 1).reshape(l, H * hd))
        off += l
    torch.cat(outs).backward(dout.float())
    for name, lo, hi in (("dq", 0, kc0), ("dk", kc0, vc0), ("dv", vc0, width)):
        assert _rel_err(dqkv[:, lo:hi], x.grad[:, lo:hi]) < 2e-2, name


@pytest.mark.gpu
def test_fused_rope_kv_append_matches_separate_ops(cuda_device):
    H, Hkv, hd = 8, 4, 128
    lens = [3, 70, 129]
    B = len(lens)
    table, kc, vc = _paged_cache(cuda_device, [l + 1 for l in lens], Hkv, hd, 16)
    kc2, vc2 = kc.clone(), vc.clone()
    ld = (H + 2 * Hkv) * hd
    qkv = torch.randn(B, ld, device=cuda_device).bfloat16()
    ref = qkv.clone()
    pos = torch.tensor(lens, device=cuda_device, dtype=torch.int32)
    slots = torch.arange(B, device=cuda_device, dtype=torch.int32)
    cos_t, sin_t = K.rope_tables(256, hd, 10000.0, cuda_device)
    K.rope_(ref, pos, cos_t, sin_t, 0, H, hd)
    K.rope_(ref, pos, cos_t, sin_t, H * hd, Hkv, hd)
    K.kv_append(ref, H * hd, (H + Hkv) * hd, slots, pos, table, kc, vc, Hkv, hd)
    K.rope_kv_append_(qkv, 0, H * hd, (H + Hkv) * hd, slots, pos, cos_t, sin_t, table, kc2, vc2, H, Hkv, hd)
    assert torch.equal(qkv, ref) and torch.equal(kc, kc2) and torch.equal(vc, vc2)
    assert kc2.abs().sum() > 0


@pytest.mark.gpu
def test_rmsnorm_wide_rows_use_the_streaming_kernel(cuda_device):
    T, d = 5, 16384        # more than 256 threads x 4 vectors: the row no longer fits in registers
    x = torch.randn(T, d, device=cuda_device).bfloat16()
    w = torch.randn(d, device=cuda_device).bfloat16()
    y, rstd, _ = K.rmsnorm_fwd(x, w, 1e-5)
    xf = x.float()
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert _rel_err(y, ref) < 1e-2


@pytest.mark.gpu
def test_flag_barrier_timeout_reports_status(cuda_device):
    """The device-side barrier gives up after its time limit and reports it in the status word; the
    context stays usable. Two 'ranks' share one pad here: rank 0 waits for a flag that nothing sets."""
    import ctypes
    from rpeg_b200.ops._lib import check, lib
    pad = torch.zeros(2048, dtype=torch.int32, device=cuda_device)
    pads = (ctypes.c_void_p * 2)(pad.data_ptr(), pad.data_ptr())
    st = K.status_word()
    st.zero_()
    stream = torch.cuda.current_stream().cuda_stream
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    check(lib().rpeg_flag_barrier(pads, 0, 2, 3, 1, None, None, 20_000_000, st.data_ptr(), stream), "rpeg_flag_barrier")
    t1.record()
    with pytest.raises(K.KernelWaitTimeout, match="code=2"):
        K.check_status()
    assert 15.0 < t0.elapsed_time(t1) < 500.0            # waited about 20 ms, not forever
    assert pad[3 * 8 + 0].item() == 1 and pad[3 * 8 + 1].item() == 0
    # the second rank arrives: its own flag is set and rank 0's flag is already there, so no timeout
    check(lib().rpeg_flag_barrier(pads, 1, 2, 3, 1, None, None, 20_000_000, st.data_ptr(), stream), "rpeg_flag_barrier")
    K.check_status()
    assert pad[3 * 8 + 1].item() == 1
    assert torch.equal(K.gemm(torch.ones(128, 64, device=cuda_device).bfloat16(), torch.ones(128, 64, device=cuda_device).bfloat16()),
                       torch.full((128, 128), 64.0, device=cuda_device).bfloat16())


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,Kd,all_reduce", [(128, 256, 64, False), (384, 1000, 520, False), (256, 4096, 2048, True)])
def test_gemm_reduce_scatter_kernel_single_rank(cuda_device, M, N, Kd, all_reduce):
    """With one rank the fused row-parallel kernel must equal a plain GEMM (its push and reduce phases
    then run against local memory only)."""
    from rpeg_b200.parallel.tp import RowParallelLinear
    x = torch.randn(M, Kd, device=cuda_device).bfloat16()
    w = (torch.randn(N, Kd, device=cuda_device) * 0.1).bfloat16()
    layer = RowParallelLinear(w, max_rows=512, device=cuda_device, all_reduce=all_reduce)
    for _ in range(2):
        y = layer.forward(x)
        K.check_status()
        assert _rel_err(y, x.float() @ w.float().t()) < 1e-2
    layer.close()


@pytest.mark.gpu
def test_headnorm_fwd_bwd(cuda_device):
    T, H, hd, col0 = 37, 6, 128, 128
    ld = col0 + H * hd + 64
    x = torch.randn(T, ld, device=cuda_device).bfloat16()
    w = (1 + 0.1 * torch.randn(hd, device=cuda_device)).bfloat16()
    dy = torch.randn(T, ld, device=cuda_device).bfloat16()
    y = x.clone()
    rstd = K.headnorm_fwd_(y, col0, H, hd, w, 1e-6)
    xr = x[:, col0:col0 + H * hd].float().view(T, H, hd).requires_grad_(True)
    wr = w.float().requires_grad_(True)
    ref = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    assert _rel_err(y[:, col0:col0 + H * hd], ref.reshape(T, -1)) < 1e-2
    assert torch.equal(y[:, :col0], x[:, :col0]) and torch.equal(y[:, col0 + H * hd:], x[:, col0 + H * hd:])
    ref.backward(dy[:, col0:col0 + H * hd].float().view(T, H, hd))
    d = dy.clone()
    dw = torch.zeros(hd, dtype=torch.float32, device=cuda_device)
    K.headnorm_bwd_(d, x, col0, H, hd, w, rstd, dw)
    assert _rel_err(d[:, col0:col0 + H * hd], xr.grad.reshape(T, -1)) < 2e-2
    assert _rel_err(dw, wr.grad) < 2e-2
    assert torch.equal(d[:, :col0], dy[:, :col0])


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,Kd", [(8, 4096, 1376), (24, 4096, 512), (40, 1536, 4096), (130, 2752, 4096), (256, 4096, 1376)])
def test_skinny_gemms_of_a_tensor_parallel_shard(cuda_device, M, N, Kd):
    """The shapes one of 8 tensor-parallel ranks works on: a contraction that is not a multiple of the 64-wide k-block
    (1376 = 11008 / 8, the last block is filled with zeros by TMA), every activation tile height (32, 64, 128 rows and two
    tiles), as split-K partials and as a plain GEMM, against fp32 PyTorch."""
    torch.manual_seed(M + N)
    ws = torch.empty(8 * 1024 * 1024, dtype=torch.float32, device=cuda_device)
    a = torch.randn(M, Kd, device=cuda_device).bfloat16()
    w = (torch.randn(N, Kd, device=cuda_device) * 0.05).bfloat16()
    want = a.float() @ w.float().t()
    parts = K.gemm_partials(a, w, ws)
    assert _rel_err(parts.reduce(), want) < 1e-2
    assert _rel_err(K.gemm(a, w, bn=128, chain=True), want) < 1e-2
    assert _rel_err(K.gemm(a, w, workspace=ws), want) < 1e-2
    K.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("M", [3, 32, 200])
def test_split_k_partials_and_their_consumers(cuda_device, M):
    d, f, H, Hkv, hd = 1024, 1408, 8, 4, 128
    ws = torch.empty(8 * 1024 * 1024, dtype=torch.float32, device=cuda_device)
    x = torch.randn(M, d, device=cuda_device).bfloat16()
    res = torch.randn(M, d, device=cuda_device).bfloat16()
    w_norm = (1 + 0.1 * torch.randn(d, device=cuda_device)).bfloat16()
    # GEMM partials sum to the GEMM
    wo = (torch.randn(d, d, device=cuda_device) * 0.05).bfloat16()
    parts = K.gemm_partials(x, wo, ws)
    assert parts.splits >= 1 and _rel_err(parts.reduce(), x.float() @ wo.float().t()) < 1e-2
    # RMSNorm over partials + residual == unfused sequence
    y, h = K.rmsnorm_fwd_partials(parts, w_norm, 1e-5, residual=res, want_sum=True)
    o_ref = K.gemm(x, wo, workspace=torch.empty_like(ws))
    y_ref, _, h_ref = K.rmsnorm_fwd(o_ref, w_norm, 1e-5, residual=res, want_sum=True)
    assert _rel_err(h, h_ref) < 1e-2 and _rel_err(y, y_ref) < 1e-2
    # SwiGLU over partials
    wgu = (torch.randn(2 * f, d, device=cuda_device) * 0.05).bfloat16()
    pg = K.gemm_partials(x, wgu, ws)
    assert _rel_err(K.swiglu_fwd_partials(pg), K.swiglu_fwd(K.gemm(x, wgu))) < 1e-2
    # RoPE + append over partials == reduce, rotate, append
    lens = [5 + (7 * i) % 100 for i in range(M)]
    table, kc, vc = _paged_cache(cuda_device, [l + 1 for l in lens], Hkv, hd, 2 * M + 8)
    kc2, vc2 = kc.clone(), vc.clone()
    wqkv = (torch.randn((H + 2 * Hkv) * hd, d, device=cuda_device) * 0.05).bfloat16()
    pos = torch.tensor(lens, device=cuda_device, dtype=torch.int32)
    slots = torch.arange(M, device=cuda_device, dtype=torch.int32)
    cos_t, sin_t = K.rope_tables(1024, hd, 10000.0, cuda_device)
    ref = K.gemm(x, wqkv)
    K.rope_kv_append_(ref, 0, H * hd, (H + Hkv) * hd, slots, pos, cos_t, sin_t, table, kc, vc, H, Hkv, hd)
    pq = K.gemm_partials(x, wqkv, ws)
    qkv = torch.zeros_like(ref)
    K.rope_kv_append_partials_(pq, qkv, 0, H * hd, (H + Hkv) * hd, slots, pos, cos_t, sin_t, table, kc2, vc2, H, Hkv, hd)
    assert _rel_err(qkv[:, :H * hd], ref[:, :H * hd]) < 1e-2
    assert _rel_err(kc2, kc) < 1e-2 and _rel_err(vc2, vc) < 1e-2
    K.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (384, 1000, 520), (256, 2048, 4096)])
def test_all_gather_gemm_kernel_single_rank(cuda_device, M, N, Kd):
    """With one rank the fused column-parallel kernel has nothing to gather and must equal a plain GEMM."""
    from rpeg_b200.parallel.tp import ColumnParallelLinear
    w = (torch.randn(N, Kd, device=cuda_device) * 0.1).bfloat16()
    layer = ColumnParallelLinear(w, max_rows=512, device=cuda_device)
    for _ in range(3):
        x = torch.randn(M, Kd, device=cuda_device).bfloat16()
        layer.input_rows(M).copy_(x)
        y = layer.forward(M)
        K.check_status()
        assert _rel_err(y, x.float() @ w.float().t()) < 1e-2
    layer.close()


@pytest.mark.gpu
def test_top_k_top_p_sampling(cuda_device):
    B, V = 64, 4000
    logits = (torch.randn(B, V, device=cuda_device) * 3).bfloat16()
    lf = logits.float()
    full_lp = torch.log_softmax(lf, -1)
    order = lf.argsort(-1, descending=True)
    # top-k: the draw stays inside the k most likely tokens; log-prob is the full-softmax one
    for seed in range(3):
        tok, lp = K.sample(logits, 1.0, False, seed, top_k=5)
        chosen = lf.gather(1, tok.long()[:, None])[:, 0]
        assert bool((chosen >= lf.gather(1, order[:, 4:5])[:, 0]).all())        # at least as large as the 5th largest logit
        assert torch.allclose(lp, full_lp.gather(1, tok.long()[:, None])[:, 0], atol=2e-2)
    # top-p: the drawn token lies inside the smallest prefix of the sorted distribution reaching the mass
    probs = full_lp.exp()
    csum = probs.gather(1, order).cumsum(-1)
    tok, _ = K.sample(logits, 1.0, False, 7, top_p=0.5)
    nucleus = ((csum < 0.5).sum(-1) + 1).clamp(max=V - 1)                    # size of the smallest prefix reaching the mass
    floor = lf.gather(1, order.gather(1, nucleus[:, None]))[:, 0]            # logit of the first token outside (ties tolerated)
    assert bool((lf.gather(1, tok.long()[:, None])[:, 0] >= floor).all())
    # k = 1 is the argmax; over many draws top-k = 3 visits only (and all of) the three best tokens of a peaked row
    tok1, _ = K.sample(logits, 1.0, False, 3, top_k=1)
    assert torch.equal(lf.gather(1, tok1.long()[:, None])[:, 0], lf.max(-1).values)   # a maximal logit (bf16 ties exist)
    row = torch.zeros(256, V, device=cuda_device)
    row[:, 10], row[:, 20], row[:, 30] = 5.0, 4.5, 4.0
    seen = set()
    for seed in range(4):
        seen |= set(K.sample(row.bfloat16(), 1.0, False, 100 + seed, top_k=3)[0].tolist())
    assert seen == {10, 20, 30}


@pytest.mark.gpu
def test_scatter_rows_by_index_single_rank(cuda_device):
    import ctypes
    n, width = 37, 24
    src = torch.randn(n, width, device=cuda_device)
    idx = torch.randperm(64, device=cuda_device)[:n].to(torch.int64)
    dst = torch.zeros(64, width, device=cuda_device)
    K.scatter_rows_by_index(src, idx, 64, (ctypes.c_void_p * 1)(dst.data_ptr()), 1)
    ref = torch.zeros_like(dst)
    ref[idx] = src
    assert torch.equal(dst, ref)


@pytest.mark.gpu
def test_version_words_publish_wait_and_gated_gemm(cuda_device):
    """Version words on one GPU (publisher and consumer in the same process, publish first): the poll sees a
    published version at once and runs out of time for one that nothing publishes; a GEMM behind an open gate
    equals the plain GEMM; a GEMM behind a gate that never opens gives up within its bound, reports the timeout
    through the status word and leaves the context usable."""
    flags = torch.zeros(8, dtype=torch.int32, device=cuda_device)
    result = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    K.publish_version([flags.data_ptr()], 0, 5)
    K.publish_version([flags.data_ptr()], 1, 5)
    K.wait_flags(flags[:2], 5, 0.05, result)
    assert result.item() == 1 and flags[:3].tolist() == [5, 5, 0]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    K.wait_flags(flags[:2], 6, 0.02, result)               # version 6 never comes: a poll that runs out, not an error
    t1.record()
    assert result.item() == 0
    assert 15.0 < t0.elapsed_time(t1) < 500.0
    K.check_status()
    g = torch.Generator(device=cuda_device).manual_seed(4)
    a = torch.randn(300, 512, device=cuda_device, generator=g).bfloat16()
    w = (torch.randn(384, 512, device=cuda_device, generator=g) * 0.05).bfloat16()
    want = K.gemm(a, w)
    got = K.gemm(a, w, gate=(flags[:2], 5, 0.5))
    assert torch.equal(want, got)
    K.check_status()
    t0.record()
    K.gemm(a, w, gate=(flags[:2], 6, 0.03))                 # closed gate: bounded wait, status word, no hang
    t1.record()
    with pytest.raises(K.KernelWaitTimeout):
        K.check_status()
    assert 20.0 < t0.elapsed_time(t1) < 1500.0
    assert torch.equal(K.gemm(a, w), want)                  # context and kernel still fine
    K.check_status()
