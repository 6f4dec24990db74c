"""GPU test of the allocation-free decode attention entry, called through its exported C symbol.

Some hosts of this library may not allocate device memory when they call it (a C serving loop with a fixed
memory budget, code that runs while the allocator is locked down); for them the split-KV attention keeps its
partial results in an array that is part of the library. The entry is compared with the regular one
(caller-provided scratch) and with an fp32 PyTorch attention on two calls in a row with different inputs, which
also shows that nothing left in the built-in scratch by the first call disturbs the second."""
import ctypes
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from rpeg_b200.ops import kernels as K  # noqa: E402

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "rpeg_b200", "librpeg_kernels.so")
P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _entry():
    lib = ctypes.CDLL(LIB)
    fn = lib.rpeg_paged_decode_attn_static
    fn.restype = I
    fn.argtypes = [P, I, I, P, P, P, I, P, P, I, I, I, I, I, F, P]
    err = lib.rpeg_static_entry_strerror
    err.restype = ctypes.c_char_p
    err.argtypes = [I]
    return fn, err


def _case(dev, lens, H, Hkv, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    hd, B = 128, len(lens)
    max_pages = (max(lens) + K.KV_PAGE - 1) // K.KV_PAGE
    n_pages = B * max_pages + 1
    table = (torch.randperm(n_pages - 1, generator=g)[: B * max_pages] + 1).view(B, max_pages).to(dev, torch.int32).contiguous()
    kc = torch.randn(n_pages, Hkv, K.KV_PAGE, hd, generator=g).bfloat16().to(dev)
    vc = torch.randn(n_pages, Hkv, K.KV_PAGE, hd, generator=g).bfloat16().to(dev)
    q = torch.randn(B, H * hd, generator=g).bfloat16().to(dev)
    seq = torch.tensor(lens, dtype=torch.int32, device=dev)
    return q, kc, vc, table, seq


def _torch_attention(q, kc, vc, table, lens, H, Hkv):
    """fp32 PyTorch oracle: softmax(q k^T / sqrt(d)) v per row over the row's pages."""
    hd, out = 128, []
    for b, l in enumerate(lens):
        pages = table[b, : (l + K.KV_PAGE - 1) // K.KV_PAGE].long()
        k = kc[pages].float().permute(1, 0, 2, 3).reshape(Hkv, -1, hd)[:, :l].repeat_interleave(H // Hkv, 0)
        v = vc[pages].float().permute(1, 0, 2, 3).reshape(Hkv, -1, hd)[:, :l].repeat_interleave(H // Hkv, 0)
        p = torch.softmax(torch.einsum("hd,hld->hl", q[b].float().view(H, hd), k) / math.sqrt(hd), -1)
        out.append(torch.einsum("hl,hld->hd", p, v).reshape(-1))
    return torch.stack(out)


def test_static_scratch_entry_matches_regular_entry_twice(cuda_device):
    fn, err = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (lens, H, Hkv, nsplit) in enumerate([([700, 65, 1, 333], 8, 8, 4), ([129, 2000, 64], 16, 4, 8)]):
        q, kc, vc, table, seq = _case(cuda_device, lens, H, Hkv, seed=10 + call)
        ref = K.paged_decode_attn(q, 0, kc, vc, table, seq, H, Hkv, 128, 1 / math.sqrt(128), nsplit=nsplit)
        out = torch.empty_like(ref)
        rc = fn(q.data_ptr(), q.stride(0), 0, kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0), seq.data_ptr(),
                out.data_ptr(), len(lens), H, Hkv, 128, nsplit, 1 / math.sqrt(128), stream)
        assert rc == 0, err(rc).decode()
        torch.cuda.synchronize()
        assert torch.equal(out, ref), f"call {call}: max diff {(out.float() - ref.float()).abs().max().item()}"
        oracle = _torch_attention(q, kc, vc, table, lens, H, Hkv)
        assert ((out.float() - oracle).abs().max() <= 1e-2 * oracle.abs().max()).item(), f"call {call} against fp32 PyTorch"
        # nsplit = 1 bypasses the scratch and must agree as well
        out1 = torch.empty_like(ref)
        assert fn(q.data_ptr(), q.stride(0), 0, kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0), seq.data_ptr(),
                  out1.data_ptr(), len(lens), H, Hkv, 128, 1, 1 / math.sqrt(128), stream) == 0
        torch.cuda.synchronize()
        assert ((out1.float() - ref.float()).abs().max() <= 2e-2 * ref.float().abs().max()).item()


def test_static_scratch_entry_refuses_what_does_not_fit(cuda_device):
    fn, err = _entry()
    q, kc, vc, table, seq = _case(cuda_device, [10, 20], 8, 8, seed=3)
    out = torch.empty_like(q)
    args = (q.data_ptr(), q.stride(0), 0, kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0), seq.data_ptr(), out.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(*args, 1024, 32, 32, 128, 8, 0.1, stream)          # 1024 * 32 * 8 partials > 16384
    assert rc == -5 and b"16384" in err(rc)
    assert fn(*args, 2, 8, 8, 128, 65, 0.1, stream) == -3 and b"nsplit" in err(-3)
    assert fn(*args, 2, 8, 3, 128, 2, 0.1, stream) == -2
    assert err(0) == b"ok"
    torch.cuda.synchronize()
    K.check_status()
