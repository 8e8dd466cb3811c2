"""Python face of the communicator.

One `Communicator` drives either this process's rank of a multi-process world
(one process per GPU, `torchrun`/`mpirun`/own launcher) or, with
`Communicator.virtual(n)`, all `n` ranks of a world emulated on a single GPU.
In the second form every tensor argument is a list with one tensor per rank.

The intended consumer is the one the reference's smoke script shows
(script/gpu_inference_test.py:21-45): `all_reduce` of fp16 activations inside
tensor-parallel inference.
"""
from __future__ import annotations

import os
import uuid
from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

import torch

from .._ext import load

TensorOrList = Union[torch.Tensor, Sequence[torch.Tensor]]

SCHED_NAMES = ["parallel", "sequential", "ring", "bisect", "oneshot", "bulk", "nvls"]
PROTO_NAMES = ["LL8", "LL16", "LL128", "LL512"]

FLAG_ROUND_EACH_ADD = 1  # sum in the element type like the reference (rt64_128.hpp:950-966)
FLAG_MUTE_SENDS = 2      # fault injection: this rank sends nothing


@dataclass
class CollInfo:
    sched: str
    proto: str
    ctas: int
    warps: int
    nwires: int
    steps: int
    first_flag: int
    launches: int
    staged: bool

    @classmethod
    def from_vec(cls, v):
        return cls(SCHED_NAMES[v[0]], PROTO_NAMES[v[1]], v[2], v[3], v[4], v[5], v[6], v[7], bool(v[8]))


class CollectiveError(RuntimeError):
    """A device-side bounded wait ran out or a peer aborted."""


def _env_rank():
    for r, w, l in (("B200IPC_RANK", "B200IPC_WORLD", "B200IPC_LOCAL_RANK"), ("RANK", "WORLD_SIZE", "LOCAL_RANK"),
                    ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK"),
                    ("PMI_RANK", "PMI_SIZE", "MPI_LOCALRANKID"), ("SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID")):
        if r in os.environ and w in os.environ:
            rank, world = int(os.environ[r]), int(os.environ[w])
            return rank, world, int(os.environ.get(l, rank))
    return 0, 1, 0


class Communicator:
    def __init__(self, handle: int, virtual: bool):
        self._C = load()
        self._h = handle
        self._virtual = virtual
        self.world = self._C.world(handle)
        self.nlocal = self._C.nlocal(handle)
        self.rank = self._C.rank(handle, 0)
        self.last_info: Optional[CollInfo] = None
        # largest input (bytes per rank) the one-shot all-reduce + residual + RMSNorm kernel is used for
        self.fused_oneshot_max_bytes = 256 << 10

    # ------------------------------------------------------------------ creation
    @classmethod
    def create(cls, rank: Optional[int] = None, world: Optional[int] = None, device: Optional[int] = None, *,
               job_id: Optional[str] = None, instance: int = 0, staging_bytes: int = 256 << 20, nvls: bool = False,
               timeout_ms: int = 2000, backing: str = "auto", device_seq: bool = False, first_seq: int = 1,
               max_ctas: int = 0, bootstrap_timeout_ms: int = 60000) -> "Communicator":
        """Collective: every rank of the job calls it.  Rank, world size and the
        device default to what the launcher put into the environment."""
        C = load()
        erank, eworld, elocal = _env_rank()
        rank = erank if rank is None else rank
        world = eworld if world is None else world
        device = elocal if device is None else device
        if job_id is None:
            job_id = os.environ.get("B200IPC_JOB_ID") or ("port" + os.environ["MASTER_PORT"] if "MASTER_PORT" in os.environ else "default")
        h = C.comm_create(rank, world, device, job_id, instance, staging_bytes, nvls, timeout_ms, backing, device_seq,
                          first_seq, max_ctas, bootstrap_timeout_ms)
        comm = cls(h, False)
        if os.environ.get("B200IPC_SELFTEST", "0") not in ("", "0") and world > 1:
            comm.self_test()  # falls back to the 8-byte-granule formats if a 64-byte segment is ever seen torn
        return comm

    @classmethod
    def from_torch_distributed(cls, device: Optional[int] = None, **kw) -> "Communicator":
        """Uses an initialised `torch.distributed` group for rank/world and to agree on a job id."""
        import torch.distributed as dist

        rank, world = dist.get_rank(), dist.get_world_size()
        token = [uuid.uuid4().hex if rank == 0 else None]
        dist.broadcast_object_list(token, src=0)
        if device is None:
            device = int(os.environ.get("LOCAL_RANK", rank))
        return cls.create(rank, world, device, job_id=token[0], **kw)

    @classmethod
    def virtual(cls, world: int, device: int = 0, *, staging_bytes: int = 64 << 20, timeout_ms: int = 2000,
                device_seq: bool = False, first_seq: int = 1, max_ctas: int = 0) -> "Communicator":
        """All `world` ranks emulated on one GPU (one cooperative launch per collective)."""
        C = load()
        h = C.comm_create_virtual(world, device, staging_bytes, timeout_ms, device_seq, first_seq, max_ctas)
        return cls(h, True)

    def close(self):
        if self._h is not None:
            self._C.comm_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------------ helpers
    def _lists(self, x: TensorOrList) -> List[torch.Tensor]:
        if isinstance(x, torch.Tensor):
            if self.nlocal != 1:
                raise ValueError(f"this communicator drives {self.nlocal} ranks: pass one tensor per rank")
            return [x]
        x = list(x)
        if len(x) != self.nlocal:
            raise ValueError(f"expected {self.nlocal} tensors, got {len(x)}")
        return x

    def _ret(self, like: TensorOrList, out: List[torch.Tensor]):
        return out[0] if isinstance(like, torch.Tensor) else out

    @staticmethod
    def _aligned(t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        if t.data_ptr() % 16:
            t = t.clone()
        return t

    # ------------------------------------------------------------------ collectives
    def all_reduce_(self, x: torch.Tensor, algo: str = "auto") -> torch.Tensor:
        """In-place sum over ranks of one contiguous, 16-byte aligned tensor: the shortest path from
        Python to the kernel (no argument normalisation, no launch report)."""
        return torch.ops.b200ipc.all_reduce_(x, self._h, algo)

    def all_reduce(self, x: TensorOrList, out: Optional[TensorOrList] = None, algo: str = "auto", *, ctas: int = 0,
                   warps: int = 0, flags: int = 0):
        """Sum over ranks.  In place unless `out` is given.  Stream-ordered on the current stream."""
        ins = self._lists(x)
        outs = ins if out is None else self._lists(out)
        fixed_in = [self._aligned(t) for t in ins]
        fixed_out = [o if (o.is_contiguous() and o.data_ptr() % 16 == 0) else torch.empty_like(o, memory_format=torch.contiguous_format)
                     for o in outs]
        if out is None:
            fixed_out = [fi if fi is i else fi for fi, i in zip(fixed_in, ins)]
        v = torch.ops.b200ipc.all_reduce(fixed_in, fixed_out, self._h, algo, ctas, warps, flags)
        for o, f in zip(outs, fixed_out):
            if o is not f:
                o.copy_(f)
        self.last_info = CollInfo.from_vec(v)
        return self._ret(x, outs)

    def all_gather(self, x: TensorOrList, out: Optional[TensorOrList] = None, algo: str = "allgather_auto", *,
                   ctas: int = 0, warps: int = 0, flags: int = 0):
        """Rank-ordered concatenation along dim 0."""
        ins = [self._aligned(t) for t in self._lists(x)]
        if out is None:
            outs = [torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device) for t in ins]
        else:
            outs = self._lists(out)
        v = torch.ops.b200ipc.all_gather(ins, outs, self._h, algo, ctas, warps, flags)
        self.last_info = CollInfo.from_vec(v)
        return self._ret(x, outs)

    def reduce_scatter(self, x: TensorOrList, out: Optional[TensorOrList] = None, algo: str = "auto", *, ctas: int = 0,
                       flags: int = 0):
        """Sum over ranks; rank r keeps the r-th of `world` equal slices along dim 0."""
        ins = [self._aligned(t) for t in self._lists(x)]
        if out is None:
            outs = [torch.empty((t.shape[0] // self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device) for t in ins]
        else:
            outs = self._lists(out)
        v = torch.ops.b200ipc.reduce_scatter(ins, outs, self._h, algo, ctas, flags)
        self.last_info = CollInfo.from_vec(v)
        return self._ret(x, outs)

    def allreduce_residual_rmsnorm(self, x: TensorOrList, residual: TensorOrList, gamma: TensorOrList, eps: float = 1e-5,
                                   *, ctas: int = 0):
        """Returns (RMSNorm(all_reduce(x) + residual) * gamma, all_reduce(x) + residual).

        Decode-sized inputs (up to 256 KiB per rank) take ONE kernel: the one-shot flag-in-data exchange with the
        add and the norm in its epilogue.  Larger ones (prefill) would push world - 1 copies of everything over the
        links that way, so they take the bandwidth-optimal all-reduce of `auto` followed by one fused add + RMSNorm
        kernel over the local result."""
        xs = self._lists(x)
        rs = self._lists(residual)
        gs = self._lists(gamma)
        xs2 = [t.reshape(-1, t.shape[-1]) for t in xs]
        rs2 = [t.reshape(-1, t.shape[-1]) for t in rs]
        if xs2[0].numel() * xs2[0].element_size() > self.fused_oneshot_max_bytes and self.world > 1:
            ins = [t.contiguous() for t in xs2]
            summed = [torch.empty_like(t) for t in ins]  # x itself is left alone
            self.all_reduce(ins if self._virtual else ins[0], summed if self._virtual else summed[0], "auto")
            pairs = [torch.ops.b200ipc.add_rmsnorm(s, r.contiguous(), g.contiguous(), eps) for s, r, g in zip(summed, rs2, gs)]
            outs = [p[0].view(t.shape) for p, t in zip(pairs, xs)]
            res_outs = [p[1].view(t.shape) for p, t in zip(pairs, xs)]
            return self._ret(x, outs), self._ret(x, res_outs)
        outs = [torch.empty_like(t) for t in xs2]
        res_outs = [torch.empty_like(t) for t in xs2]
        v = torch.ops.b200ipc.fused_ar_rmsnorm(xs2, rs2, gs, outs, res_outs, eps, self._h, ctas)
        self.last_info = CollInfo.from_vec(v)
        outs = [o.view(t.shape) for o, t in zip(outs, xs)]
        res_outs = [o.view(t.shape) for o, t in zip(res_outs, xs)]
        return self._ret(x, outs), self._ret(x, res_outs)

    def allreduce_scale_cast(self, x: TensorOrList, scale: float = 1.0, dtype: Optional[torch.dtype] = None, *,
                             ctas: int = 0):
        """cast(all_reduce(x) * scale) from one kernel."""
        xs = [self._aligned(t) for t in self._lists(x)]
        outs = [torch.empty_like(t, dtype=dtype or t.dtype) for t in xs]
        v = torch.ops.b200ipc.fused_ar_scale_cast(xs, outs, scale, self._h, ctas)
        self.last_info = CollInfo.from_vec(v)
        return self._ret(x, outs)

    @staticmethod
    def pack_weight(weight: torch.Tensor) -> torch.Tensor:
        """Re-lays a row-parallel weight [N, K] (nn.Linear layout, N a multiple of 64) for `linear_allreduce`:
        [N / 64, K blocks, 64, 64], every 64 x 64 block stored as the 128-byte-swizzled shared-memory image the
        tensor core reads (16-byte chunk c of row r sits at chunk c ^ (r % 8)), K zero-padded to a multiple of
        256.  Done once at load time; the kernel then streams the weight with one contiguous bulk copy per
        stage, which is worth most at decode sizes where the layer is bound by reading the weight."""
        N, K = weight.shape
        if N % 64:
            raise ValueError("pack_weight needs N to be a multiple of 64")
        kb = (K + 255) // 256 * 4
        wp = torch.zeros(N, kb * 64, dtype=weight.dtype, device=weight.device)
        wp[:, :K] = weight
        blocks = wp.view(N // 64, 64, kb, 8, 8).permute(0, 2, 1, 3, 4)  # [row block, k block, row, chunk, element]
        r = torch.arange(64, device=weight.device) % 8
        c = torch.arange(8, device=weight.device)
        src_chunk = (c[None, :] ^ r[:, None])[None, None, :, :, None].expand(N // 64, kb, 64, 8, 8)
        return torch.gather(blocks, 3, src_chunk).contiguous().view(N // 64, kb, 64, 64)

    def linear_allreduce(self, x: TensorOrList, weight: TensorOrList, residual: Optional[TensorOrList] = None,
                         gamma: Optional[TensorOrList] = None, eps: float = 1e-5, *, ctas: int = 0,
                         fused: Optional[bool] = None):
        """Row-parallel linear layer fused with its all-reduce in one tcgen05/TMA kernel.

        fused=None picks by size: between 33 and 256 rows on four or more GPUs the framework's matmul followed by
        `allreduce_residual_rmsnorm` measured ahead of the single kernel (8 GPUs, 128 rows: 40 us against 53 us),
        so that pair runs there (plain weights with residual and gamma only); everything else takes the kernel.

        x: [M, K_local], weight: [N, K_local] (nn.Linear layout) of this rank, or that weight packed once by
        `pack_weight` (faster, most of all at decode sizes).  Returns
        `y = all_reduce(x @ weight.T)` when neither residual nor gamma is given, else the pair
        `(RMSNorm(y + residual) * gamma, y + residual)`.  Outputs live in the symmetric heap; calls of one shape
        alternate between two sets of them, so a result stays valid through the next call of that shape (it may
        be that call's residual) and is overwritten by the one after."""
        xs = [t.contiguous() for t in self._lists(x)]
        ws = [t.contiguous() for t in self._lists(weight)]
        M, N = xs[0].shape[0], ws[0].shape[0] * (64 if ws[0].dim() == 4 else 1)  # 4-D: packed by pack_weight
        if fused is None:
            fused = not (32 < M <= 256 and self.world >= 4 and not self._virtual and ws[0].dim() == 2
                         and residual is not None and gamma is not None)
        if not fused:
            part = [a @ w.t() for a, w in zip(xs, ws)]
            return self.allreduce_residual_rmsnorm(part if self._virtual else part[0], residual, gamma, eps)
        key = (M, N, xs[0].dtype)
        cache = self.__dict__.setdefault("_gemm_buffers", {})
        if key not in cache:
            nbytes = self._C.gemm_ar_workspace_bytes(self.world, M, N)
            wsp = self.empty([nbytes // 2], torch.float16)
            for t in (wsp if self._virtual else [wsp]):
                t.zero_()
            torch.cuda.synchronize()
            self.barrier()  # nobody may push into a workspace that its owner is still clearing
            # two sets of outputs, used in turn: the `res_out` of one call can be the `residual` of the next
            cache[key] = [wsp, [(self.empty([M, N], xs[0].dtype), self.empty([M, N], xs[0].dtype)) for _ in range(2)], 0]
        entry = cache[key]
        wsp, (out, res_out) = entry[0], entry[1][entry[2]]
        entry[2] ^= 1
        L = (lambda t: t) if self._virtual else (lambda t: [t])
        with_norm = gamma is not None
        want_res = residual is not None
        v = torch.ops.b200ipc.fused_gemm_ar(xs, ws, self._lists(residual) if want_res else [], self._lists(gamma) if with_norm else [],
                                            L(out), L(res_out) if want_res else [], L(wsp), eps, with_norm, self._h, ctas, False)
        self.last_info = CollInfo.from_vec(v)
        if with_norm or want_res:
            return out, res_out
        return out

    def linear(self, x: TensorOrList, weight: TensorOrList, *, ctas: int = 0):
        """`x @ weight.T` with no exchange: the column-parallel projections of a decode step (QKV, gate/up) on the
        same weight-streaming tcgen05 kernel that `linear_allreduce` uses for up to 32 rows (swapped operands,
        split K, all SMs pulling on the weight).  x: [M <= 32, K], weight: [N, K] with N a multiple of 128, or
        packed by `pack_weight`; anything else goes to the framework's matmul.  The output lives in the symmetric
        heap and is reused by the next call with the same shape."""
        xs = [t.contiguous() for t in self._lists(x)]
        ws = [t.contiguous() for t in self._lists(weight)]
        M, N = xs[0].shape[0], ws[0].shape[0] * (64 if ws[0].dim() == 4 else 1)
        if M > 32 or N % 128 != 0 or xs[0].shape[1] % 8 != 0:
            if ws[0].dim() == 4:
                raise ValueError("a packed weight needs M <= 32 rows and N a multiple of 128")
            return self._ret(x, [a @ w.t() for a, w in zip(xs, ws)])
        key = ("local", M, N, xs[0].dtype)
        cache = self.__dict__.setdefault("_gemm_buffers", {})
        if key not in cache:
            nbytes = self._C.gemm_ar_workspace_bytes(self.world, M, N)
            wsp = self.empty([nbytes // 2], torch.float16)
            for t in (wsp if self._virtual else [wsp]):
                t.zero_()
            torch.cuda.synchronize()
            cache[key] = (wsp, self.empty([M, N], xs[0].dtype))
        wsp, out = cache[key]
        L = (lambda t: t) if self._virtual else (lambda t: [t])
        v = torch.ops.b200ipc.fused_gemm_ar(xs, ws, [], [], L(out), [], L(wsp), 0.0, False, self._h, ctas, True)
        self.last_info = CollInfo.from_vec(v)
        return out

    def allgather_linear(self, x_shard: TensorOrList, weight: TensorOrList, *, ctas: int = 0, fused: Optional[bool] = None):
        """Column-parallel linear layer on row-sharded activations, all-gather fused into the GEMM kernel.

        fused=None picks by size: the fused kernel from 4096 gathered rows up (level with cuBLAS + NCCL at 8192
        rows on 8 GPUs); below that this library's all-gather followed by the framework's matmul, which measured
        ahead of both the fused kernel and NCCL + cuBLAS (128 rows: 49 us against 60 and 55).

        x_shard: [M / world, K] (this rank's rows), weight: [N_local, K].  Returns `concat(x_shards) @ weight.T`,
        shape [M, N_local]: every rank pushes its rows to all ranks and the tcgen05/TMA GEMM starts on the rows
        that are already there while the others arrive."""
        xs = [t.contiguous() for t in self._lists(x_shard)]
        ws = [t.contiguous() for t in self._lists(weight)]
        M, K, N = xs[0].shape[0] * self.world, xs[0].shape[1], ws[0].shape[0]
        if fused is None:
            fused = M >= 4096 or self.world == 1
        if not fused:
            gathered = self.all_gather(xs if self._virtual else xs[0], None, "allgather_auto")
            gs = gathered if self._virtual else [gathered]
            return self._ret(x_shard, [g.view(M, K) @ w.t() for g, w in zip(gs, ws)])
        cache = self.__dict__.setdefault("_ag_buffers", {})
        key = (M, K)
        if key not in cache:
            cache[key] = self.empty([2 * (M * K + 128)], xs[0].dtype)
            torch.cuda.synchronize()
            self.barrier()
        wsp = cache[key]
        outs = [torch.empty(M, N, dtype=t.dtype, device=t.device) for t in xs]
        v = torch.ops.b200ipc.fused_ag_gemm(xs, ws, outs, wsp if self._virtual else [wsp], self._h, ctas)
        self.last_info = CollInfo.from_vec(v)
        return self._ret(x_shard, outs)

    # ------------------------------------------------------------------ symmetric memory
    def empty(self, shape, dtype=torch.float16):
        """A tensor inside the symmetric heap (same offset on every rank): the large-message
        collectives then work on it without staging.  Every rank must allocate in the same order."""
        shape = list(shape) if not isinstance(shape, int) else [shape]
        ts = [self._C.sym_empty(self._h, shape, dtype, i) for i in range(self.nlocal)]
        return ts if self._virtual else ts[0]

    def free_symmetric(self):
        """Releases every symmetric allocation at once.  Tensors handed out by `empty()` before, and the
        outputs of earlier `linear_allreduce` / `allgather_linear` calls (whose cached workspaces live in
        the same region), become invalid: the next allocations reuse their memory."""
        self.__dict__.pop("_gemm_buffers", None)
        self.__dict__.pop("_ag_buffers", None)
        self._C.sym_free_all(self._h)

    # ------------------------------------------------------------------ state
    @property
    def has_nvls(self) -> bool:
        return self._C.has_nvls(self._h)

    @property
    def nvls_note(self) -> str:
        return self._C.nvls_note(self._h)

    @property
    def backing(self) -> str:
        return self._C.backing(self._h)

    @property
    def launches(self) -> int:
        return self._C.launches(self._h)

    def status(self, local: int = 0):
        keys = ("code", "rank", "peer", "wire", "step", "expected", "seen", "where")
        return dict(zip(keys, self._C.status(self._h, local)))

    def check(self):
        """Raises CollectiveError if any finished collective recorded a failure.  Call after a stream sync."""
        try:
            self._C.raise_if_failed(self._h)
        except RuntimeError as e:
            raise CollectiveError(str(e)) from None

    def reset(self):
        """After a failed collective: waits for the device, clears rings, flags and the status (collective
        in a multi-process world).  The cached workspaces of the fused GEMM kernels are cleared too, so that
        no flag left by an interrupted launch can be taken for a later one."""
        self._C.reset(self._h)
        for entry in self.__dict__.get("_gemm_buffers", {}).values():
            for t in (entry[0] if self._virtual else [entry[0]]):
                t.zero_()
        torch.cuda.synchronize()
        self.barrier()

    def barrier(self):
        self._C.host_barrier(self._h)

    def set_timeout_ms(self, ms: int):
        self._C.set_timeout_ms(self._h, ms)

    def set_thresholds(self, oneshot_max_bytes: int, ll_max_bytes: int):
        self._C.set_thresholds(self._h, oneshot_max_bytes, ll_max_bytes)

    def set_seq(self, seq: int):
        self._C.set_seq(self._h, seq)

    @property
    def seq(self) -> int:
        return self._C.seq(self._h)

    def state_dict(self) -> dict:
        """What a job has to carry over a checkpoint: the flag sequence number (rings of a fresh communicator are
        zero, so any later sequence number is safe), the algorithm cut-offs and the safe-format switch.  The
        reference keeps the same single piece of state in its `-f` flag (main.cpp:185 there)."""
        return {"seq": int(self.seq), "world": int(self.world), "safe_protocols": bool(self.safe_protocols)}

    def load_state_dict(self, state: dict) -> None:
        if int(state.get("world", self.world)) != self.world:
            raise ValueError(f"checkpoint is from a world of {state['world']}, this communicator has {self.world} ranks")
        self.set_seq(int(state["seq"]))
        if state.get("safe_protocols"):
            self._C.set_safe_protos(self._h, True)

    # ------------------------------------------------------------------ protocol safety
    def soak(self, algos=("simple_pcie_p", "simple", "small_pcie_p", "small"), min_transactions: int = 100000,
             nelems: int = 1 << 20) -> dict:
        """Bit-exact stress of the flag-in-data wire formats on this communicator's links: all-reduces of the
        reference's integer pattern (i % 32) * (rank + 1) in fp16 (every partial sum exact), refilled before every
        launch, until each algorithm has moved at least `min_transactions` warp transactions per rank; every
        result element must equal the known sum exactly.  Returns {algo: {"transactions", "launches",
        "mismatches"}}.  LL128 / LL512 (`simple*`) carry one flag per 64-byte segment and rely on such a segment
        arriving whole - the assumption the reference flags at rt64_128.hpp:544; this is the test of it."""
        i = torch.arange(nelems, device="cuda") % 32
        world = self.world
        want = (i * sum(r + 1 for r in range(world))).to(torch.float16)
        ranks = [self._C.rank(self._h, k) for k in range(self.nlocal)]
        pats = [(i * (r + 1)).to(torch.float16) for r in ranks]
        report = {}
        for algo in algos:
            bad = torch.zeros((), dtype=torch.int64, device="cuda")
            bufs = [torch.empty_like(p) for p in pats]
            done = launches = 0
            while done < min_transactions:
                for b, p in zip(bufs, pats):
                    b.copy_(p)
                self.all_reduce(bufs if self._virtual else bufs[0], None, algo)
                for b in bufs:
                    bad += (b != want).sum()
                done += int(self.last_info.steps) * int(self.last_info.nwires)
                launches += 1
            torch.cuda.synchronize()
            self.check()
            report[algo] = {"transactions": done, "launches": launches, "mismatches": int(bad)}
        return report

    def self_test(self, min_transactions: int = 20000) -> bool:
        """Short soak of the two 64-byte-segment formats.  If a single element ever differs, `auto` stops using
        them on this communicator (8-byte-granule formats only) and False is returned.  Collective."""
        rep = self.soak(("simple_pcie_p", "simple"), min_transactions, nelems=1 << 18)
        ok = all(v["mismatches"] == 0 for v in rep.values())
        if self.world > 1 and not self._virtual:
            import torch.distributed as dist

            if dist.is_initialized():
                t = torch.tensor([0 if ok else 1], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ok = int(t.item()) == 0
        self._C.set_safe_protos(self._h, not ok)
        return ok

    @property
    def safe_protocols(self) -> bool:
        return self._C.safe_protos(self._h)

    # ------------------------------------------------------------------ device-side trace
    def set_trace(self, on: bool = True):
        """Every completed device-side wait of the flag-in-data kernels leaves a time-stamped record (wire, site,
        peer, step, flag) in a ring inside the rank's heap; `B200IPC_DEBUG=1` in the environment switches it on
        at creation.  The analogue of the reference's verbose build (allreduce.hpp:96-101)."""
        self._C.set_trace_wires(self._h, on)

    def trace_events(self, local: int = 0):
        """The records of the trace ring, oldest first: dicts with t_ns, wire, site, peer, step, flag, rank, and
        the total number of records written so far (the ring keeps the most recent ones)."""
        off, entries, rec = self._C.trace_ring(self._h)
        raw = self.dump_heap(off, 16 + entries * rec, local)
        total = int(raw[:4].view(torch.int32)[0]) & 0xFFFFFFFF
        body = raw[16:].view(torch.int64).view(entries, rec // 8)
        n = min(total, entries)
        first = total % entries if total > entries else 0
        out = []
        for k in range(n):
            row = body[(first + k) % entries]
            words = row[1:].contiguous().view(torch.int32).tolist()
            out.append(dict(t_ns=int(row[0]), wire=words[0], site=words[1], peer=words[2], step=words[3],
                            flag=words[4] & 0xFFFFFFFF, rank=words[5]))
        return out, total

    def heap_layout(self):
        keys = ("ctrl_off", "scatter_off", "gather_off", "half_bytes", "oneshot_off", "oneshot_bytes", "staging_off",
                "staging_bytes", "total_bytes")
        return dict(zip(keys, self._C.heap_layout(self._h)))

    def dump_heap(self, offset: int, nbytes: int, local: int = 0) -> torch.Tensor:
        """Host copy of a piece of this rank's heap (debug view of the scratch rings)."""
        return self._C.dump_heap(self._h, local, offset, nbytes)
