"""GPU numerics of the entropy bonus: the entropy kernel and the combined log-prob + entropy backward against PyTorch
fp32 autograd on the same bf16 logits, and a policy step whose loss moves by ``-entropy_coef * mean entropy``."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from rpeg_b200.engine import algorithms as A  # noqa: E402
from rpeg_b200.models.llama import LlamaConfig, LlamaModel  # noqa: E402
from rpeg_b200.ops import kernels as K  # noqa: E402


@pytest.mark.parametrize("V, temperature", [(1000, 1.0), (1003, 0.7)])
def test_entropy_kernels_match_autograd(cuda_device, V, temperature):
    g = torch.Generator(device="cpu").manual_seed(5)
    T, ld = 6, (V + 7) // 8 * 8
    orig = (torch.randn(T, ld, generator=g) * 2.0).bfloat16().to(cuda_device)      # rows padded to a multiple of 8 elements
    store = orig.clone()
    logits = store[:, :V]
    targets = torch.randint(0, V, (T,), generator=g, dtype=torch.int32).to(cuda_device)
    coef = torch.randn(T, generator=g).to(cuda_device)
    ecoef = torch.randn(T, generator=g).to(cuda_device)
    x = (logits.float() / temperature).requires_grad_(True)
    logp = torch.log_softmax(x, dim=-1)
    ent_ref = -(logp.exp() * logp).sum(-1)
    lp, lse = K.token_logprob_fwd(logits, targets, temperature)
    ent = K.token_entropy(logits, lse, temperature)
    assert torch.allclose(ent, ent_ref.detach(), atol=2e-3, rtol=1e-3)
    loss = (coef * logp[torch.arange(T), targets.long()]).sum() + (ecoef * ent_ref).sum()
    loss.backward()
    want = x.grad / temperature                                   # d loss / d logits
    got = K.token_logprob_entropy_bwd_(logits, targets, lse, coef, ent, ecoef, temperature).float()   # in place
    assert (got - want).abs().max() <= 1e-2 * want.abs().max() + 1e-4
    # with a zero entropy coefficient the combined kernel writes what the plain one writes
    a, b = orig.clone(), orig.clone()
    K.token_logprob_bwd_(a[:, :V], targets, lse, coef, temperature)
    K.token_logprob_entropy_bwd_(b[:, :V], targets, lse, coef, ent, torch.zeros_like(ecoef), temperature)
    assert torch.equal(a[:, :V], b[:, :V])
    K.check_status()


def test_policy_step_with_entropy_bonus(cuda_device):
    """The loss reported with ``entropy_coef = c`` is the loss without it minus ``c`` times the mean token entropy, and
    the bonus changes the gradient."""
    cfg = LlamaConfig.tiny(n_layers=2)
    g = torch.Generator().manual_seed(9)
    N, S, T = 6, 10, 12
    prompts = torch.randint(3, cfg.vocab, (N, S), generator=g, dtype=torch.int32).to(cuda_device)
    resp = torch.randint(3, cfg.vocab, (N, T), generator=g, dtype=torch.int32).to(cuda_device)
    lens = [int(v) for v in torch.randint(4, T + 1, (N,), generator=g)]
    mask = (torch.arange(T, device=cuda_device)[None, :] < torch.tensor(lens, device=cuda_device)[:, None]).float()
    out = {}
    for c in (0.0, 0.05):
        model = LlamaModel(cfg, cuda_device, trainable=True, seed=2)
        algo = A.AlgoConfig(micro_tokens=512, head_chunk=32, entropy_coef=c)
        ro = A.Rollout(prompts, [S] * N, resp, lens, torch.zeros((N, T), device=cuda_device), mask)
        ro.old_logp = A.sequence_logprobs(model, ro, algo)
        ro.adv = (torch.randn((N, T), generator=g).to(cuda_device) if c == 0.0 else out["adv"]) * mask
        out.setdefault("adv", ro.adv.clone())
        model.zero_grad()
        m = A.policy_train_step(model, ro, algo)
        torch.cuda.synchronize()
        out[c] = (float(m["loss"]), float(m["entropy_sum"]), model.g.clone())
    K.check_status()
    n_tok = float(sum(lens))
    (l0, e0, g0), (l1, e1, g1) = out[0.0], out[0.05]
    assert e0 == 0.0 and e1 > 0.0                                   # entropies are only computed when the bonus is on
    assert 0.0 < e1 / n_tok < torch.log(torch.tensor(float(cfg.vocab))).item() + 1e-3
    assert l1 == pytest.approx(l0 - 0.05 * e1 / n_tok, abs=2e-3)
    assert (g1 - g0).abs().max() > 0
