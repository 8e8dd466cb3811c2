"""Tiny Llama-shaped tensor-parallel decoder on an emulated world (one GPU): the two fused
all-reduce paths must reproduce a dense fp32 re-computation from the assembled weights."""
import pytest
import torch

from gpu_ipc_example_b200 import Communicator
from gpu_ipc_example_b200.models.llama import LlamaConfig, LlamaTP, dense_decode_reference

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fusion", ["allreduce", "gemm"])
@pytest.mark.parametrize("world", [2, 8])
def test_tiny_decoder_matches_dense_reference(world, fusion):
    cfg = LlamaConfig.tiny()
    B, steps = 4, 3
    with Communicator.virtual(world, 0, staging_bytes=64 << 20) as comm:
        model = LlamaTP(cfg, comm, batch=B, max_ctx=8, fusion=fusion, seed=1)
        g = torch.Generator(device="cuda").manual_seed(5)
        toks = [torch.randint(0, cfg.vocab, (B,), device="cuda", generator=g) for _ in range(steps)]
        hidden = []
        for t in toks:
            nxt = model.decode(t)
            torch.cuda.synchronize()
            comm.check()
            assert nxt.shape == (B,) and int(nxt.min()) >= 0 and int(nxt.max()) < cfg.vocab
            hidden.append([x.float().clone() for x in model.last_hidden])
        ref = dense_decode_reference(model, toks)
        for got, want in zip(hidden, ref):
            for x in got:
                torch.testing.assert_close(x, want, atol=6e-2, rtol=5e-2)
            for x in got[1:]:
                assert torch.equal(x, got[0]), "every rank must hold the same activations"


@pytest.mark.parametrize("fusion,pack", [("allreduce", False), ("gemm", True)])
def test_decoder_with_the_decode_kernels(fusion, pack):
    """head_dim 128, two query heads per KV head: RoPE + cache append, attention and SiLU * up run in the
    hand-written kernels (and, for the fused GEMM, on packed weights); same dense fp32 reference."""
    cfg = LlamaConfig.tiny128()
    B, steps, world = 3, 5, 2
    with Communicator.virtual(world, 0, staging_bytes=64 << 20) as comm:
        model = LlamaTP(cfg, comm, batch=B, max_ctx=8, fusion=fusion, seed=2, pack_weights=pack)
        assert model.kernels
        g = torch.Generator(device="cuda").manual_seed(11)
        toks = [torch.randint(0, cfg.vocab, (B,), device="cuda", generator=g) for _ in range(steps)]
        hidden = []
        for t in toks:
            model.decode(t)
            torch.cuda.synchronize()
            comm.check()
            hidden.append([x.float().clone() for x in model.last_hidden])
        ref = dense_decode_reference(model, toks)
        for got, want in zip(hidden, ref):
            for x in got:
                torch.testing.assert_close(x, want, atol=6e-2, rtol=5e-2)
            assert torch.equal(got[0], got[1]), "every rank must hold the same activations"
