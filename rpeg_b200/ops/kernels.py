"""Thin tensor-level wrappers over the native sm_100a kernels (no autograd here).

Every wrapper validates shapes/dtypes/contiguity on the host, passes raw device pointers plus the
current CUDA stream to the C ABI in ``csrc/rpeg_kernels.h`` and raises on a non-zero return code.
Kernels with bounded waits share one per-device status word; ``check_status()`` reads it (this
synchronises) and raises ``KernelWaitTimeout`` if any wait ran out. With ``RPEG_CHECK_ARGS=1`` the wrappers also
validate the index VALUES held by tensor arguments before the launch (``ops/checked.py``).
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import checked as _chk
from ._lib import check, lib

KV_PAGE = 64
MAX_PEERS = 8
_status: dict[int, torch.Tensor] = {}


class KernelWaitTimeout(RuntimeError):
    """A bounded device-side wait (mbarrier or peer flag) ran out; the kernel returned early."""


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def status_word(device: torch.device | None = None) -> torch.Tensor:
    dev = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if dev not in _status:
        _status[dev] = torch.zeros(4, dtype=torch.int32, device=f"cuda:{dev}")
    return _status[dev]


def check_status() -> None:
    """Read the status word of the current device (synchronises) and raise if a wait timed out."""
    st = status_word()
    vals = st.tolist()
    if vals[0] != 0:
        st.zero_()
        raise KernelWaitTimeout(f"device wait timed out: code={vals[0]} where={vals[1]} block={vals[2]} extra={vals[3]}")


def _req(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if not t.is_cuda or t.dtype != dtype:
        raise TypeError(f"{name}: expected a CUDA {dtype} tensor, got {t.dtype} on {t.device}")


# --------------------------------------------------------------------------- GEMM
GEMM_CHAIN = 0x1000     # flag in the tile-width argument of rpeg_gemm_bf16: launch as a programmatic dependent


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False,
         bn: int = 0, workspace: torch.Tensor | None = None, gate: tuple | None = None, chain: bool = False) -> torch.Tensor:
    """``C[M,N] = op(a) @ op(b).T`` on tcgen05 tensor cores with fp32 accumulation.

    ``gate = (flags uint32 tensor, min_version, timeout_s)`` holds back every operand load until all words of
    ``flags`` reached ``min_version`` (weights being pushed into ``b`` by other GPUs); the wait is bounded.

    ``a`` is ``[M,K]`` (or ``[K,M]`` with ``trans_a``); ``b`` is ``[N,K]`` — the ``[out,in]`` layout
    of a linear weight — or ``[K,N]`` with ``trans_b``. Rows may be strided (last dim contiguous).
    ``out_dtype=float32, accumulate=True`` adds into ``out`` (used for weight-gradient accumulation).
    ``workspace`` (fp32 scratch) lets skinny problems (M <= 256, e.g. decode) run split-K so every SM
    streams part of the weight matrix. ``chain``: the call is a link of a decode step whose kernels are launched as
    programmatic dependents (``b`` is a weight matrix that no kernel of the step writes): the grid may start under the
    previous kernel's tail and fetch weight tiles before that kernel has finished.
    """
    _req(a, torch.bfloat16, "a")
    _req(b, torch.bfloat16, "b")
    if a.dim() != 2 or b.dim() != 2 or a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("gemm operands must be 2-D with a contiguous last dimension")
    M, K = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if trans_b else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm inner dimensions differ: {K} vs {Kb}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an `out` tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        out_dtype = out.dtype
        if out.shape != (M, N) or out.stride(1) != 1:
            raise ValueError("gemm out has the wrong shape or a strided last dimension")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("gemm output must be bf16 or fp32")
    if M == 0 or N == 0:
        return out
    if gate is not None:
        flags, min_version, timeout_s = gate
        rc = lib().rpeg_gemm_bf16_gated(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                        out.stride(0), int(trans_a), int(trans_b), int(out_dtype == torch.float32),
                                        int(accumulate), bn, _ptr(workspace), 0 if workspace is None else workspace.numel(),
                                        flags.data_ptr(), flags.numel(), int(min_version), int(timeout_s * 1e9),
                                        status_word(a.device).data_ptr(), _stream())
        check(rc, "rpeg_gemm_bf16_gated")
        return out
    rc = lib().rpeg_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                              out.stride(0), int(trans_a), int(trans_b), int(out_dtype == torch.float32),
                              int(accumulate), bn | (GEMM_CHAIN if chain else 0), _ptr(workspace), 0 if workspace is None else workspace.numel(),
                              status_word(a.device).data_ptr(), _stream())
    check(rc, "rpeg_gemm_bf16")
    return out


def gemm_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``silu(x @ W_gate.T) * (x @ W_up.T)`` with ``w_gate_up = [W_gate; W_up]`` of shape ``[2f, K]``: the gated MLP's first
    linear with the activation applied to the fp32 accumulators in the GEMM epilogue, so the ``[M, 2f]`` pre-activation is
    never written. ``f`` must be a multiple of 128 (callers fall back to ``gemm`` + ``swiglu_fwd`` otherwise)."""
    _req(x, torch.bfloat16, "x")
    _req(w_gate_up, torch.bfloat16, "w_gate_up")
    M, Kd = x.shape
    f = w_gate_up.shape[0] // 2
    if w_gate_up.shape[1] != Kd or x.stride(1) != 1 or w_gate_up.stride(1) != 1:
        raise ValueError("gemm_swiglu: x [M, K] and w_gate_up [2f, K] must share K and be contiguous in it")
    if f % 128:
        raise ValueError("gemm_swiglu needs d_ff to be a multiple of 128")
    if out is None:
        out = torch.empty((M, f), dtype=torch.bfloat16, device=x.device)
    if M == 0:
        return out
    check(lib().rpeg_gemm_swiglu(x.data_ptr(), w_gate_up.data_ptr(), out.data_ptr(), M, f, Kd, x.stride(0), w_gate_up.stride(0),
                                 out.stride(0), status_word(x.device).data_ptr(), _stream()), "rpeg_gemm_swiglu")
    return out


def set_pdl(on: bool) -> None:
    """Programmatic dependent launches for the kernels launched from now on (a captured graph keeps its setting)."""
    lib().rpeg_set_pdl(int(bool(on)))


def publish_version(flag_ptrs, word: int, version: int) -> None:
    """After the copies queued on this stream: store ``version`` into word ``word`` of every flag array in
    ``flag_ptrs`` (device pointers, local or peer) with system-scope release."""
    arr = (ctypes.c_void_p * len(flag_ptrs))(*[int(p) for p in flag_ptrs])
    check(lib().rpeg_publish_version(arr, len(flag_ptrs), int(word), int(version), _stream()), "rpeg_publish_version")


def wait_flags(flags: torch.Tensor, min_version: int, timeout_s: float, result: torch.Tensor) -> None:
    """``result[0] = 1`` (int32) once all words of ``flags`` reached ``min_version``, ``0`` if ``timeout_s`` ran out first."""
    check(lib().rpeg_wait_flags(flags.data_ptr(), flags.numel(), int(min_version), int(timeout_s * 1e9), result.data_ptr(), _stream()),
          "rpeg_wait_flags")


# --------------------------------------------------------------------------- norm / rope / swiglu
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
                want_sum: bool = False):
    """Returns ``(y, rstd, h)``: ``h = x + residual`` (only when asked for), ``y = rmsnorm(h) * w``."""
    _req(x, torch.bfloat16, "x")
    T, d = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    h = torch.empty_like(x) if (residual is not None and want_sum) else None
    check(lib().rpeg_rmsnorm_fwd(x.data_ptr(), _ptr(residual), w.data_ptr(), _ptr(h), y.data_ptr(),
                                 rstd.data_ptr(), T, d, eps, _stream()), "rpeg_rmsnorm_fwd")
    return y, rstd, h


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor, dw: torch.Tensor,
                dres_in: torch.Tensor | None = None) -> torch.Tensor:
    """``dx`` of ``y = rmsnorm(x) * w`` (+ ``dres_in`` added in); accumulates ``dw`` (fp32) in place."""
    T, d = x.shape
    dx = torch.empty_like(x)
    check(lib().rpeg_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), _ptr(dres_in),
                                 dx.data_ptr(), dw.data_ptr(), T, d, _stream()), "rpeg_rmsnorm_bwd")
    return dx


def rope_tables(max_pos: int, head_dim: int, theta: float, device, scaling_factor: float = 1.0,
                original_max_pos: int = 8192) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables ``[max_pos, head_dim/2]``. ``scaling_factor > 1`` applies the llama3 frequency
    scaling (low_freq_factor 1, high_freq_factor 4): long wavelengths are divided by the factor, short
    ones kept, the band in between interpolated."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    if scaling_factor > 1.0:
        low, high = 1.0, 4.0
        wavelen = 2 * math.pi / inv
        smooth = ((original_max_pos / wavelen) - low) / (high - low)
        mid = (1 - smooth) * inv / scaling_factor + smooth * inv
        inv = torch.where(wavelen > original_max_pos / low, inv / scaling_factor,
                          torch.where(wavelen < original_max_pos / high, inv, mid))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


def rope_(buf: torch.Tensor, pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor, col0: int, nheads: int,
          head_dim: int, backward: bool = False) -> None:
    """Rotate ``nheads`` heads starting at column ``col0`` of the 2-D ``buf`` in place."""
    _req(buf, torch.bfloat16, "buf")
    if _chk.active():
        _chk.rope("rpeg_rope", pos, buf.shape[0], cos_t)
    check(lib().rpeg_rope(buf.data_ptr(), pos.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), buf.shape[0],
                          buf.stride(0), col0, nheads, head_dim, int(backward), _stream()), "rpeg_rope")


def headnorm_fwd_(buf: torch.Tensor, col0: int, nheads: int, head_dim: int, w: torch.Tensor, eps: float,
                  want_rstd: bool = True) -> torch.Tensor | None:
    """RMS-normalise every (row, head) slice of ``buf[:, col0 : col0 + nheads*head_dim]`` in place with the
    shared weight ``w [head_dim]`` (QK-norm). Returns ``rstd [T, nheads]`` for the backward pass."""
    _req(buf, torch.bfloat16, "buf")
    T = buf.shape[0]
    rstd = torch.empty((T, nheads), dtype=torch.float32, device=buf.device) if want_rstd else None
    check(lib().rpeg_headnorm_fwd(buf.data_ptr(), buf.stride(0), col0, nheads, head_dim, w.data_ptr(), _ptr(rstd), T, eps,
                                  _stream()), "rpeg_headnorm_fwd")
    return rstd


def headnorm_bwd_(dbuf: torch.Tensor, x_pre: torch.Tensor, col0: int, nheads: int, head_dim: int, w: torch.Tensor,
                  rstd: torch.Tensor, dw: torch.Tensor) -> None:
    """In place on ``dbuf`` (dy -> dx) for the slices normalised by ``headnorm_fwd_``; ``x_pre`` holds the
    pre-norm values in the same column layout; ``dw [head_dim]`` fp32 is accumulated."""
    check(lib().rpeg_headnorm_bwd(dbuf.data_ptr(), dbuf.stride(0), x_pre.data_ptr(), x_pre.stride(0), col0, nheads, head_dim,
                                  w.data_ptr(), rstd.data_ptr(), dw.data_ptr(), dbuf.shape[0], _stream()), "rpeg_headnorm_bwd")


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    T, f2 = gu.shape
    out = torch.empty((T, f2 // 2), dtype=gu.dtype, device=gu.device)
    check(lib().rpeg_swiglu_fwd(gu.data_ptr(), out.data_ptr(), T, f2 // 2, _stream()), "rpeg_swiglu_fwd")
    return out


def swiglu_bwd(gu: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    T, f2 = gu.shape
    dgu = torch.empty_like(gu)
    check(lib().rpeg_swiglu_bwd(gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), T, f2 // 2, _stream()),
          "rpeg_swiglu_bwd")
    return dgu


def add_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    out = torch.empty_like(a) if out is None else out
    check(lib().rpeg_add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _stream()), "rpeg_add_bf16")
    return out


def embed_fwd(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _req(ids, torch.int32, "ids")
    if _chk.active():
        _chk.embed("rpeg_embed_fwd", ids, table.shape[0])
    if out is None:
        out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    elif out.shape != (ids.numel(), table.shape[1]) or not out.is_contiguous() or out.dtype != table.dtype:
        raise ValueError("embed_fwd: `out` must be a contiguous [tokens, d] tensor of the table's dtype")
    check(lib().rpeg_embed_fwd(ids.data_ptr(), table.data_ptr(), out.data_ptr(), ids.numel(), table.shape[1],
                               _stream()), "rpeg_embed_fwd")
    return out


def embed_bwd(ids: torch.Tensor, dout: torch.Tensor, dtable: torch.Tensor) -> None:
    if _chk.active():
        _chk.embed("rpeg_embed_bwd", ids, dtable.numel() // dout.shape[1])
    check(lib().rpeg_embed_bwd(ids.data_ptr(), dout.data_ptr(), dtable.data_ptr(), ids.numel(), dout.shape[1],
                               _stream()), "rpeg_embed_bwd")


# --------------------------------------------------------------------------- losses
def token_logprob_fwd(logits: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0):
    _req(logits, torch.bfloat16, "logits")
    _req(targets, torch.int32, "targets")
    T, V = logits.shape
    logp = torch.empty(T, dtype=torch.float32, device=logits.device)
    lse = torch.empty(T, dtype=torch.float32, device=logits.device)
    check(lib().rpeg_token_logprob_fwd(logits.data_ptr(), targets.data_ptr(), logp.data_ptr(), lse.data_ptr(), T, V,
                                       logits.stride(0), temperature, _stream()), "rpeg_token_logprob_fwd")
    return logp, lse


def token_logprob_bwd_(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, coef: torch.Tensor,
                       temperature: float = 1.0) -> torch.Tensor:
    """Overwrite ``logits`` with ``d loss / d logits`` given ``coef = d loss / d logp`` per row."""
    T, V = logits.shape
    check(lib().rpeg_token_logprob_bwd(logits.data_ptr(), targets.data_ptr(), lse.data_ptr(), coef.data_ptr(), T, V,
                                       logits.stride(0), temperature, _stream()), "rpeg_token_logprob_bwd")
    return logits


def token_entropy(logits: torch.Tensor, lse: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """Entropy of every row's softmax (at ``temperature``) from the logits and the log-sum-exp ``token_logprob_fwd`` returned."""
    _req(logits, torch.bfloat16, "logits")
    T, V = logits.shape
    ent = torch.empty(T, dtype=torch.float32, device=logits.device)
    check(lib().rpeg_token_entropy(logits.data_ptr(), lse.data_ptr(), ent.data_ptr(), T, V, logits.stride(0), temperature, _stream()),
          "rpeg_token_entropy")
    return ent


def token_logprob_entropy_bwd_(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, coef: torch.Tensor, ent: torch.Tensor,
                               ecoef: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """Overwrite ``logits`` with ``d loss / d logits`` given ``coef = d loss / d logp`` and ``ecoef = d loss / d entropy`` per row."""
    T, V = logits.shape
    check(lib().rpeg_token_logprob_entropy_bwd(logits.data_ptr(), targets.data_ptr(), lse.data_ptr(), coef.data_ptr(), ent.data_ptr(),
                                               ecoef.data_ptr(), T, V, logits.stride(0), temperature, _stream()),
          "rpeg_token_logprob_entropy_bwd")
    return logits


def policy_loss(lp, old_lp, ref_lp, adv, mask, clip_eps: float, kl_coef: float, inv_denom: float):
    """Clipped PPO/GRPO loss. Returns ``(coef, acc)``; ``acc = [loss, sum(lp-ref), n_clipped, sum(old-lp)]``."""
    coef = torch.empty_like(lp)
    acc = torch.zeros(4, dtype=torch.float32, device=lp.device)
    check(lib().rpeg_policy_loss(lp.data_ptr(), old_lp.data_ptr(), _ptr(ref_lp), adv.data_ptr(), mask.data_ptr(),
                                 coef.data_ptr(), acc.data_ptr(), lp.numel(), clip_eps, kl_coef, inv_denom,
                                 _stream()), "rpeg_policy_loss")
    return coef, acc


def masked_rowsum(x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    B, T = x.shape
    out = torch.empty(B, dtype=torch.float32, device=x.device)
    check(lib().rpeg_masked_rowsum(x.data_ptr(), mask.data_ptr(), out.data_ptr(), B, T, _stream()),
          "rpeg_masked_rowsum")
    return out


def dpo_loss(pi_seq: torch.Tensor, ref_seq: torch.Tensor, beta: float):
    """Rows interleaved (chosen, rejected). Returns ``(seq_coef, acc)``; ``acc = [loss, n_correct, margin]``."""
    P = pi_seq.numel() // 2
    seq_coef = torch.empty_like(pi_seq)
    acc = torch.zeros(4, dtype=torch.float32, device=pi_seq.device)
    check(lib().rpeg_dpo_loss(pi_seq.data_ptr(), ref_seq.data_ptr(), seq_coef.data_ptr(), acc.data_ptr(), P, beta,
                              _stream()), "rpeg_dpo_loss")
    return seq_coef, acc


def expand_seq_coef(seq_coef: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    B, T = mask.shape
    coef = torch.empty_like(mask)
    check(lib().rpeg_expand_seq_coef(seq_coef.data_ptr(), mask.data_ptr(), coef.data_ptr(), B, T, _stream()),
          "rpeg_expand_seq_coef")
    return coef


def value_loss(v, ret, mask, inv_denom: float):
    dv = torch.empty_like(v)
    acc = torch.zeros(4, dtype=torch.float32, device=v.device)
    check(lib().rpeg_value_loss(v.data_ptr(), ret.data_ptr(), mask.data_ptr(), dv.data_ptr(), acc.data_ptr(),
                                v.numel(), inv_denom, _stream()), "rpeg_value_loss")
    return dv, acc


def gae(old_lp, ref_lp, values, mask, scores, beta: float, gamma: float, lam: float, whiten: bool):
    B, T = values.shape
    adv = torch.empty_like(values)
    ret = torch.empty_like(values)
    check(lib().rpeg_gae(old_lp.data_ptr(), _ptr(ref_lp), values.data_ptr(), mask.data_ptr(), scores.data_ptr(),
                         adv.data_ptr(), ret.data_ptr(), B, T, beta, gamma, lam, int(whiten), _stream()), "rpeg_gae")
    return adv, ret


def group_advantage(rewards: torch.Tensor, group: int) -> torch.Tensor:
    out = torch.empty_like(rewards)
    check(lib().rpeg_group_advantage(rewards.data_ptr(), out.data_ptr(), rewards.numel() // group, group, _stream()),
          "rpeg_group_advantage")
    return out


def sample(logits: torch.Tensor, temperature: float, greedy: bool, seed: int, forced: torch.Tensor | None = None,
           token_out: torch.Tensor | None = None, logp_out: torch.Tensor | None = None,
           seed_offset: torch.Tensor | None = None, top_k: int = 0, top_p: float = 1.0):
    """Gumbel-max sample (or argmax) per row with its log-prob; ``seed_offset`` is an int64 device
    scalar mixed into the seed so graph replays draw fresh noise. ``top_k`` / ``top_p`` restrict the draw to
    the k most likely tokens / the smallest set reaching mass ``top_p``; the log-prob is under the full softmax."""
    B, V = logits.shape
    tok = torch.empty(B, dtype=torch.int32, device=logits.device) if token_out is None else token_out
    lp = torch.empty(B, dtype=torch.float32, device=logits.device) if logp_out is None else logp_out
    if not greedy and (0 < top_k < V or top_p < 1.0):
        check(lib().rpeg_sample_filtered(logits.data_ptr(), B, V, logits.stride(0), temperature, int(top_k), float(top_p),
                                         seed & 0xFFFFFFFFFFFFFFFF, _ptr(seed_offset), _ptr(forced), tok.data_ptr(), lp.data_ptr(),
                                         _stream()), "rpeg_sample_filtered")
        return tok, lp
    check(lib().rpeg_sample(logits.data_ptr(), B, V, logits.stride(0), temperature, int(greedy),
                            seed & 0xFFFFFFFFFFFFFFFF, _ptr(seed_offset), _ptr(forced), tok.data_ptr(), lp.data_ptr(),
                            _stream()),
          "rpeg_sample")
    return tok, lp


def head_gemv(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    T, d = h.shape
    out = torch.empty(T, dtype=torch.float32, device=h.device)
    check(lib().rpeg_head_gemv(h.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), T, d, _stream()),
          "rpeg_head_gemv")
    return out


def head_gemv_bwd(h, w, dout, dw: torch.Tensor, db: torch.Tensor | None) -> torch.Tensor:
    T, d = h.shape
    dh = torch.empty_like(h)
    check(lib().rpeg_head_gemv_bwd(h.data_ptr(), w.data_ptr(), dout.data_ptr(), dh.data_ptr(), dw.data_ptr(),
                                   _ptr(db), T, d, _stream()), "rpeg_head_gemv_bwd")
    return dh


# --------------------------------------------------------------------------- optimizer
def adamw_(p32, m, v, grad, w16, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, step=1, grad_scale=1.0,
           sumsq: torch.Tensor | None = None, max_norm: float = 0.0) -> None:
    n = p32.numel()
    check(lib().rpeg_adamw(p32.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(), w16.data_ptr(), n, lr,
                           beta1, beta2, eps, wd, step, grad_scale, _ptr(sumsq),
                           0 if sumsq is None else sumsq.numel(), max_norm, _stream()), "rpeg_adamw")


def sumsq(x: torch.Tensor, out: torch.Tensor) -> None:
    check(lib().rpeg_sumsq(x.data_ptr(), x.numel(), out.data_ptr(), _stream()), "rpeg_sumsq")


# --------------------------------------------------------------------------- split-K partials and their consumers
class Partials:
    """fp32 split-K partial products ``[splits, M, N]`` living in a workspace: ``sum(0)`` is the GEMM result."""

    __slots__ = ("buf", "splits", "M", "N")

    def __init__(self, buf: torch.Tensor, splits: int, M: int, N: int):
        self.buf, self.splits, self.M, self.N = buf, splits, M, N

    @property
    def stride(self) -> int:
        return self.M * self.N

    def reduce(self) -> torch.Tensor:
        return self.buf[: self.splits * self.stride].view(self.splits, self.M, self.N).sum(0)


def gemm_partials(a: torch.Tensor, b: torch.Tensor, workspace: torch.Tensor) -> Partials:
    """``a [M,K] @ b [N,K]^T`` for skinny ``M`` (decode): returns the split-K partials in ``workspace`` instead
    of reducing them; ``rmsnorm_fwd_partials`` / ``swiglu_fwd_partials`` / ``rope_kv_append_partials_`` add them
    up while loading. The split count is fixed by the shapes, so the call is CUDA-graph friendly."""
    _req(a, torch.bfloat16, "a")
    _req(b, torch.bfloat16, "b")
    M, Kd = a.shape
    N = b.shape[0]
    splits = ctypes.c_int(1)
    check(lib().rpeg_gemm_bf16_partials(a.data_ptr(), b.data_ptr(), M, N, Kd, a.stride(0), b.stride(0), workspace.data_ptr(),
                                        workspace.numel(), ctypes.byref(splits), status_word(a.device).data_ptr(), _stream()),
          "rpeg_gemm_bf16_partials")
    return Partials(workspace, int(splits.value), M, N)


def rmsnorm_fwd_partials(parts: Partials, w: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
                         want_sum: bool = False):
    """``y = rmsnorm(sum(parts) [+ residual]) * w``; with ``want_sum`` also returns the bf16 sum (the new residual stream)."""
    y = torch.empty((parts.M, parts.N), dtype=torch.bfloat16, device=w.device)
    h = torch.empty_like(y) if want_sum else None
    check(lib().rpeg_rmsnorm_fwd_partials(parts.buf.data_ptr(), parts.splits, parts.stride, _ptr(residual), w.data_ptr(), _ptr(h),
                                          y.data_ptr(), parts.M, parts.N, eps, _stream()), "rpeg_rmsnorm_fwd_partials")
    return y, h


def swiglu_fwd_partials(parts: Partials) -> torch.Tensor:
    f = parts.N // 2
    out = torch.empty((parts.M, f), dtype=torch.bfloat16, device=parts.buf.device)
    check(lib().rpeg_swiglu_fwd_partials(parts.buf.data_ptr(), parts.splits, parts.stride, out.data_ptr(), parts.M, f, _stream()),
          "rpeg_swiglu_fwd_partials")
    return out


def rope_kv_append_partials_(parts: Partials, qkv: torch.Tensor, q_col0, k_col0, v_col0, seq_id, pos, cos_t, sin_t, page_table,
                             kcache, vcache, n_heads, n_kv_heads, head_dim) -> None:
    """Sum the partials of a QKV projection, rotate q and k, store q into ``qkv`` (bf16, the attention
    kernel's query input) and k, v into the paged cache."""
    if _chk.active():
        _chk.kv_append("rpeg_rope_kv_append_partials", parts.M, seq_id, pos, page_table, kcache, n_kv_heads, head_dim, cos_t)
    check(lib().rpeg_rope_kv_append_partials(parts.buf.data_ptr(), parts.splits, parts.stride, qkv.data_ptr(), qkv.stride(0), q_col0,
                                             k_col0, v_col0, seq_id.data_ptr(), pos.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(),
                                             page_table.data_ptr(), page_table.stride(0), kcache.data_ptr(), vcache.data_ptr(),
                                             parts.M, n_heads, n_kv_heads, head_dim, _stream()), "rpeg_rope_kv_append_partials")


def scatter_rows_by_index(src: torch.Tensor, global_idx: torch.Tensor, rows_per_rank: int, dst_ptr_array, world: int) -> None:
    """Send every row of ``src [n, ...]`` to the rank owning its global index (``idx // rows_per_rank``), slot
    ``idx % rows_per_rank`` of that rank's symmetric buffer (``dst_ptr_array`` = ctypes ``void*[world]``)."""
    n = src.shape[0]
    row_bytes = src[0].numel() * src.element_size() if n else 0
    if _chk.active():
        _chk.global_rows("rpeg_scatter_rows_by_index", global_idx, rows_per_rank, world)
    check(lib().rpeg_scatter_rows_by_index(src.data_ptr(), n, row_bytes, global_idx.data_ptr(), rows_per_rank, dst_ptr_array, world,
                                           _stream()), "rpeg_scatter_rows_by_index")


# --------------------------------------------------------------------------- attention
def kv_append(qkv, k_col0, v_col0, seq_id, pos, page_table, kcache, vcache, n_kv_heads, head_dim) -> None:
    if _chk.active():
        _chk.kv_append("rpeg_kv_append", qkv.shape[0], seq_id, pos, page_table, kcache, n_kv_heads, head_dim)
    check(lib().rpeg_kv_append(qkv.data_ptr(), qkv.stride(0), k_col0, v_col0, seq_id.data_ptr(), pos.data_ptr(),
                               page_table.data_ptr(), page_table.stride(0), kcache.data_ptr(), vcache.data_ptr(),
                               qkv.shape[0], n_kv_heads, head_dim, _stream()), "rpeg_kv_append")


def rope_kv_append_(qkv, q_col0, k_col0, v_col0, seq_id, pos, cos_t, sin_t, page_table, kcache, vcache, n_heads, n_kv_heads,
                    head_dim) -> None:
    """Rotate the query and key heads of ``qkv`` in place and write the rotated keys and the values
    into the paged cache: one launch instead of two rotations and an append."""
    _req(qkv, torch.bfloat16, "qkv")
    if _chk.active():
        _chk.kv_append("rpeg_rope_kv_append", qkv.shape[0], seq_id, pos, page_table, kcache, n_kv_heads, head_dim, cos_t)
    check(lib().rpeg_rope_kv_append(qkv.data_ptr(), qkv.stride(0), q_col0, k_col0, v_col0, seq_id.data_ptr(), pos.data_ptr(),
                                    cos_t.data_ptr(), sin_t.data_ptr(), page_table.data_ptr(), page_table.stride(0),
                                    kcache.data_ptr(), vcache.data_ptr(), qkv.shape[0], n_heads, n_kv_heads, head_dim,
                                    _stream()), "rpeg_rope_kv_append")


def decode_scratch_numel(B: int, H: int, nsplit: int) -> int:
    return int(lib().rpeg_decode_attn_scratch_bytes(B, H, nsplit)) // 4


_GROUP_TC = False


def set_group_tc(on: bool) -> None:
    """Which group kernel ``paged_decode_attn(groups=...)`` uses when the caller does not say: the tcgen05 one or the
    CUDA-core one (the default)."""
    global _GROUP_TC
    _GROUP_TC = bool(on)


def paged_decode_attn(q, q_col0, kcache, vcache, page_table, seq_lens, n_heads, n_kv_heads, head_dim, scale,
                      nsplit: int = 1, scratch: torch.Tensor | None = None, out: torch.Tensor | None = None, groups=None,
                      group_tc: bool | None = None):
    """``groups = (group_rows [B, 8] int32, group_shared [B] int32, row_key0 [B] int32)``: rows that alias their first
    KV pages in groups (K samples of one prompt); the shared keys are then read once per group (``scratch`` must
    hold ``nsplit + 1`` partials per row and head). ``group_tc``: score the groups on the tensor cores (tcgen05, keys on
    the M axis) instead of the CUDA-core kernel."""
    B = q.shape[0]
    if _chk.active():
        _chk.paged_attention("rpeg_paged_decode_attn", B, seq_lens, page_table, kcache, n_kv_heads, head_dim)
    out = torch.empty((B, n_heads * head_dim), dtype=torch.bfloat16, device=q.device) if out is None else out
    if groups is not None:
        group_rows, group_shared, row_key0 = groups
        if scratch is None:
            scratch = torch.empty(decode_scratch_numel(B, n_heads, nsplit + 1), dtype=torch.float32, device=q.device)
        if _GROUP_TC if group_tc is None else group_tc:
            check(lib().rpeg_paged_decode_attn_grouped_tc(q.data_ptr(), q.stride(0), q_col0, kcache.data_ptr(), vcache.data_ptr(),
                                                          kcache.shape[0], page_table.data_ptr(), page_table.stride(0),
                                                          seq_lens.data_ptr(), out.data_ptr(), scratch.data_ptr(), B, n_heads,
                                                          n_kv_heads, head_dim, nsplit, scale, group_rows.data_ptr(),
                                                          group_shared.data_ptr(), row_key0.data_ptr(),
                                                          status_word(q.device).data_ptr(), _stream()),
                  "rpeg_paged_decode_attn_grouped_tc")
            return out
        check(lib().rpeg_paged_decode_attn_grouped(q.data_ptr(), q.stride(0), q_col0, kcache.data_ptr(), vcache.data_ptr(),
                                                   page_table.data_ptr(), page_table.stride(0), seq_lens.data_ptr(), out.data_ptr(),
                                                   scratch.data_ptr(), B, n_heads, n_kv_heads, head_dim, nsplit, scale,
                                                   group_rows.data_ptr(), group_shared.data_ptr(), row_key0.data_ptr(), _stream()),
              "rpeg_paged_decode_attn_grouped")
        return out
    if nsplit > 1 and scratch is None:
        scratch = torch.empty(decode_scratch_numel(B, n_heads, nsplit), dtype=torch.float32, device=q.device)
    check(lib().rpeg_paged_decode_attn(q.data_ptr(), q.stride(0), q_col0, kcache.data_ptr(), vcache.data_ptr(),
                                       page_table.data_ptr(), page_table.stride(0), seq_lens.data_ptr(),
                                       out.data_ptr(), _ptr(scratch), B, n_heads, n_kv_heads, head_dim, nsplit,
                                       scale, _stream()), "rpeg_paged_decode_attn")
    return out


def flash_attn_fwd(qkv, q_col0, k_col0, v_col0, cu_seqlens, max_seqlen, n_heads, n_kv_heads, head_dim, scale=None):
    """Causal attention over packed sequences. Returns ``(out [T, H*hd] bf16, lse [H, T] fp32)``."""
    _req(qkv, torch.bfloat16, "qkv")
    T = qkv.shape[0]
    if _chk.active():
        _chk.packed_sequences("rpeg_flash_attn_fwd", cu_seqlens, T, max_seqlen)
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    lse = torch.empty((n_heads, T), dtype=torch.float32, device=qkv.device)
    check(lib().rpeg_flash_attn_fwd(qkv.data_ptr(), qkv.stride(0), q_col0, k_col0, v_col0, cu_seqlens.data_ptr(),
                                    cu_seqlens.numel() - 1, max_seqlen, T, n_heads, n_kv_heads, head_dim, scale,
                                    out.data_ptr(), lse.data_ptr(), status_word(qkv.device).data_ptr(), _stream()),
          "rpeg_flash_attn_fwd")
    return out, lse


def flash_attn_bwd(qkv, q_col0, k_col0, v_col0, out, dout, lse, cu_seqlens, max_seqlen, n_heads, n_kv_heads, head_dim,
                   scale=None, dqkv: torch.Tensor | None = None) -> torch.Tensor:
    """Gradient of ``flash_attn_fwd`` w.r.t. the packed qkv buffer (same column blocks). ``dqkv``
    may be passed in to reuse a buffer; columns outside the three blocks are left untouched."""
    T = qkv.shape[0]
    if _chk.active():
        _chk.packed_sequences("rpeg_flash_attn_bwd", cu_seqlens, T, max_seqlen)
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    if dqkv is None:
        dqkv = torch.empty_like(qkv)
    dvec = torch.empty((n_heads, T), dtype=torch.float32, device=qkv.device)
    dq_acc = torch.empty((T, n_heads * head_dim), dtype=torch.float32, device=qkv.device)
    check(lib().rpeg_flash_attn_bwd(qkv.data_ptr(), qkv.stride(0), q_col0, k_col0, v_col0, out.data_ptr(),
                                    dout.data_ptr(), lse.data_ptr(), cu_seqlens.data_ptr(), cu_seqlens.numel() - 1,
                                    max_seqlen, T, n_heads, n_kv_heads, head_dim, scale, dvec.data_ptr(),
                                    dq_acc.data_ptr(), dqkv.data_ptr(), dqkv.stride(0),
                                    status_word(qkv.device).data_ptr(), _stream()), "rpeg_flash_attn_bwd")
    return dqkv


# --------------------------------------------------------------------------- decode bookkeeping
def decode_prepare(active, gen_count, forced_len, forced, eos: int) -> None:
    check(lib().rpeg_decode_prepare(active.data_ptr(), gen_count.data_ptr(), _ptr(forced_len), forced.data_ptr(),
                                    active.numel(), eos, _stream()), "rpeg_decode_prepare")


def decode_advance(sampled, sampled_lp, token, pos, seq_len, active, gen_count, out_tok, out_lp, eos: int,
                   n_finished, step_counter=None) -> None:
    check(lib().rpeg_decode_advance(sampled.data_ptr(), sampled_lp.data_ptr(), token.data_ptr(), pos.data_ptr(),
                                    seq_len.data_ptr(), active.data_ptr(), gen_count.data_ptr(), out_tok.data_ptr(),
                                    out_lp.data_ptr(), active.numel(), out_tok.shape[1], eos, n_finished.data_ptr(),
                                    _ptr(step_counter), _stream()), "rpeg_decode_advance")


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    if _chk.active():
        _chk.row_indices("rpeg_gather_rows", rows, x.shape[0])
    out = torch.empty((rows.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    check(lib().rpeg_gather_rows(x.data_ptr(), rows.data_ptr(), out.data_ptr(), rows.numel(), x.shape[1], _stream()),
          "rpeg_gather_rows")
    return out


def scatter_rows_(x: torch.Tensor, rows: torch.Tensor, src: torch.Tensor, overwrite: bool = False) -> None:
    if _chk.active():
        _chk.row_indices("rpeg_scatter_rows", rows, x.shape[0])
    check(lib().rpeg_scatter_rows(x.data_ptr(), rows.data_ptr(), src.data_ptr(), rows.numel(), x.shape[1],
                                  int(overwrite), _stream()), "rpeg_scatter_rows")
