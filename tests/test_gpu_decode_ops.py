"""The decode-step kernels (rotary embedding + KV-cache append, attention of one new token over the cache,
SiLU(gate) * up) against plain PyTorch fp32 references of the same operations."""
import math

import pytest
import torch
import torch.nn.functional as F

from gpu_ipc_example_b200._ext import load

pytestmark = pytest.mark.gpu


def _rope_ref(x, pos, theta):
    B, H, D = x.shape
    half = D // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, device=x.device, dtype=torch.float32) / half))
    ang = float(pos) * inv
    cos, sin = ang.cos(), ang.sin()
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rope_kv_append(dtype):
    load()
    B, hq, hkv, D, ctx, pos, theta = 5, 8, 2, 128, 16, 11, 5e5
    g = torch.Generator(device="cuda").manual_seed(0)
    qkv = torch.randn(B, (hq + 2 * hkv) * D, device="cuda", generator=g).to(dtype)
    kc = torch.zeros(B, hkv, ctx, D, device="cuda", dtype=dtype)
    vc = torch.zeros_like(kc)
    q0, k0, v0 = qkv.clone().split([hq * D, hkv * D, hkv * D], dim=-1)
    torch.ops.b200ipc.rope_kv_append(qkv, kc, vc, hq, hkv, pos, theta)
    torch.cuda.synchronize()
    tol = dict(atol=2e-3, rtol=2e-3) if dtype == torch.float16 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(qkv[:, :hq * D].float().view(B, hq, D), _rope_ref(q0.view(B, hq, D), pos, theta), **tol)
    torch.testing.assert_close(kc[:, :, pos].float(), _rope_ref(k0.view(B, hkv, D), pos, theta), **tol)
    assert torch.equal(vc[:, :, pos], v0.view(B, hkv, D))
    assert float(kc[:, :, :pos].abs().max()) == 0 and float(kc[:, :, pos + 1:].abs().max()) == 0


@pytest.mark.parametrize("G", [1, 2, 4, 8])
@pytest.mark.parametrize("ctx,splits", [(1, 1), (7, 2), (130, 3), (2048, 8), (1000, 32)])
def test_decode_attention(G, ctx, splits):
    C = load()
    B, hkv, D, max_ctx = 3, 2, 128, 2048
    hq = hkv * G
    g = torch.Generator(device="cuda").manual_seed(ctx * 10 + G)
    qkv = torch.randn(B, (hq + 2 * hkv) * D, device="cuda", generator=g).half()
    kc = torch.randn(B, hkv, max_ctx, D, device="cuda", generator=g).half()
    vc = torch.randn(B, hkv, max_ctx, D, device="cuda", generator=g).half()
    ws = torch.zeros(C.attention_workspace_bytes(B, hq, hkv, splits), dtype=torch.uint8, device="cuda")
    for rep in range(2):  # the second call finds the arrival counters the first one left behind
        out = torch.ops.b200ipc.decode_attention(qkv, kc, vc, ws, hq, hkv, ctx, splits)
        torch.cuda.synchronize()
        q = qkv[:, :hq * D].view(B, hq, 1, D).float()
        ref = F.scaled_dot_product_attention(q, kc[:, :, :ctx].float(), vc[:, :, :ctx].float(), enable_gqa=G > 1)
        torch.testing.assert_close(out.float().view(B, hq, D), ref.view(B, hq, D), atol=4e-3, rtol=4e-3)


def test_decode_attention_bf16_and_default_splits():
    C = load()
    B, hq, hkv, D, ctx = 32, 8, 1, 128, 2048
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B, (hq + 2 * hkv) * D, device="cuda", generator=g).bfloat16()
    kc = torch.randn(B, hkv, ctx, D, device="cuda", generator=g).bfloat16()
    vc = torch.randn(B, hkv, ctx, D, device="cuda", generator=g).bfloat16()
    splits = C.attention_splits(B, hkv, ctx, 0)
    assert 1 <= splits <= 32
    ws = torch.zeros(C.attention_workspace_bytes(B, hq, hkv, splits), dtype=torch.uint8, device="cuda")
    out = torch.ops.b200ipc.decode_attention(qkv, kc, vc, ws, hq, hkv, ctx, splits)
    q = qkv[:, :hq * D].view(B, hq, 1, D).float()
    ref = F.scaled_dot_product_attention(q, kc.float(), vc.float(), enable_gqa=True)
    torch.testing.assert_close(out.float().view(B, hq, D), ref.view(B, hq, D), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_silu_mul(dtype):
    load()
    g = torch.Generator(device="cuda").manual_seed(1)
    gu = torch.randn(33, 2 * 3584, device="cuda", generator=g).to(dtype)
    act = torch.ops.b200ipc.silu_mul(gu)
    gate, up = gu.float().split(3584, dim=-1)
    tol = dict(atol=4e-3, rtol=4e-3) if dtype == torch.float16 else dict(atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(act.float(), F.silu(gate) * up, **tol)


@pytest.mark.parametrize("dtype,hidden", [(torch.float16, 8192), (torch.bfloat16, 1024), (torch.float16, 8 * 4 * 256 + 64)])
def test_add_rmsnorm(dtype, hidden):
    load()
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(37, hidden, device="cuda", generator=g).to(dtype)
    r = torch.randn(37, hidden, device="cuda", generator=g).to(dtype)
    gam = (torch.rand(hidden, device="cuda", generator=g) + 0.5).to(dtype)
    out, res = torch.ops.b200ipc.add_rmsnorm(x, r, gam, 1e-5)
    s = (x.float() + r.float()).to(dtype).float()
    tol = dict(atol=1e-2, rtol=1e-2) if dtype == torch.float16 else dict(atol=6e-2, rtol=4e-2)
    torch.testing.assert_close(res.float(), s, atol=0, rtol=0)
    torch.testing.assert_close(out.float(), s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * gam.float(), **tol)


def test_allreduce_residual_rmsnorm_prefill_sized():
    """Above the one-shot limit the call becomes an all-reduce plus one fused add + RMSNorm kernel; same result."""
    from gpu_ipc_example_b200 import Communicator

    world, rows, hidden = 4, 512, 2048  # 2 MiB per rank
    with Communicator.virtual(world, 0, staging_bytes=64 << 20) as comm:
        g = torch.Generator(device="cuda").manual_seed(5)
        parts = [torch.randn(rows, hidden, device="cuda", generator=g).half() for _ in range(world)]
        keep = [p.clone() for p in parts]
        res = torch.randn(rows, hidden, device="cuda", generator=g).half()
        gam = (torch.rand(hidden, device="cuda", generator=g) + 0.5).half()
        out, new_res = comm.allreduce_residual_rmsnorm(parts, [res] * world, [gam] * world, 1e-5)
        torch.cuda.synchronize()
        comm.check()
        assert all(torch.equal(a, b) for a, b in zip(parts, keep)), "the inputs must not be modified"
        s = (torch.stack([p.float() for p in parts]).sum(0).half().float() + res.float()).half().float()
        torch.testing.assert_close(new_res[2].float(), s, atol=2e-2, rtol=4e-3)
        torch.testing.assert_close(out[2].float(), s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * gam.float(), atol=3e-2, rtol=1e-2)
