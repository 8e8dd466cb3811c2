"""Host-side bootstrap without a GPU: the Unix-socket mesh (byte all-gather, SCM_RIGHTS descriptor
passing, barrier, deadlines), the launcher-environment adapter, the -l device list and the algorithm
names of the CLI."""
import multiprocessing as mp
import os
import time

import pytest

from gpu_ipc_example_b200._ext import load


def _mesh_rank(rank, world, job, q):
    try:
        C = load()
        blob = bytes([rank]) * 5
        all_bytes, seen, mx = C.mesh_selftest(rank, world, job, 3, 20000, blob)
        q.put((rank, all_bytes, list(seen), mx, None))
    except Exception as e:  # noqa: BLE001
        q.put((rank, None, None, None, repr(e)))


@pytest.mark.parametrize("world", [2, 5, 8])
def test_mesh_allgather_and_fd_passing(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    job = f"pytest-{os.getpid()}-{world}-{time.time_ns()}"
    procs = [ctx.Process(target=_mesh_rank, args=(r, world, job, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    want_bytes = b"".join(bytes([r]) * 5 for r in range(world))
    for rank, all_bytes, seen, mx, err in results:
        assert err is None, err
        assert all_bytes == want_bytes
        assert seen == list(range(world))  # every received descriptor leads to its sender's memfd
        assert mx == (world - 1) * 10


def test_missing_peer_hits_the_deadline_instead_of_spinning_forever():
    C = load()
    t0 = time.time()
    with pytest.raises(RuntimeError, match="never opened its bootstrap socket|deadline"):
        C.mesh_selftest(1, 2, f"nobody-{time.time_ns()}", 0, 300, b"x")  # rank 0 never shows up
    assert time.time() - t0 < 10


def test_socket_names_keep_rank_and_instance_apart():
    C = load()
    # the reference concatenates rank and instance digits (ipc_exchange.cpp:164,178): 1|12 == 11|2 there
    assert C.socket_name("job", 12, 1) != C.socket_name("job", 2, 11)
    assert C.socket_name("a", 0, 0) != C.socket_name("b", 0, 0)


@pytest.mark.parametrize("env,want", [
    ({"RANK": "3", "WORLD_SIZE": "8", "LOCAL_RANK": "3", "MASTER_PORT": "2950"}, (3, 8, 3, "port2950")),
    ({"OMPI_COMM_WORLD_RANK": "1", "OMPI_COMM_WORLD_SIZE": "2", "OMPI_COMM_WORLD_LOCAL_RANK": "1"}, (1, 2, 1, "default")),
    ({"PMI_RANK": "5", "PMI_SIZE": "8", "MPI_LOCALRANKID": "5"}, (5, 8, 5, "default")),  # Intel MPI, as in the reference's script
    ({"SLURM_PROCID": "2", "SLURM_NTASKS": "4", "SLURM_LOCALID": "2", "SLURM_JOB_ID": "77"}, (2, 4, 2, "slurm77")),
    ({"B200IPC_RANK": "0", "B200IPC_WORLD": "2", "B200IPC_JOB_ID": "x", "RANK": "9", "WORLD_SIZE": "10"}, (0, 2, 0, "x")),
])
def test_rank_environment_adapter(monkeypatch, env, want):
    for k in list(os.environ):
        if k.split("_")[0] in ("RANK", "WORLD", "LOCAL", "OMPI", "PMI", "PMIX", "MPI", "SLURM", "B200IPC", "MASTER"):
            monkeypatch.delenv(k, raising=False)
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    found, rank, world, local, job = load().rank_env()
    assert found and (rank, world, local, job) == want


def test_device_list_option():
    C = load()
    assert C.device_for_rank("012345678", 3, 8) == 3      # the reference's default -l string
    assert C.device_for_rank("76543210", 0, 8) == 7
    assert C.device_for_rank("4,5,6,7", 2, 8) == 6
    with pytest.raises(RuntimeError, match="no entry"):
        C.device_for_rank("01", 2, 8)
    with pytest.raises(RuntimeError, match="visible"):
        C.device_for_rank("0123", 3, 2)


def test_algorithm_names():
    C = load()
    ref = {"small": ("parallel", "LL8"), "simple": ("parallel", "LL128"), "small_pcie_p": ("parallel", "LL16"),
           "simple_pcie_p": ("parallel", "LL512"), "bisect": ("bisect", "LL128"), "small_ring": ("ring", "LL16"),
           "simple_ring": ("ring", "LL512"), "small_pcie": ("sequential", "LL16"), "simple_pcie": ("sequential", "LL512")}
    for name, (sched, proto) in ref.items():
        ok, ag, auto, s, p, direct = C.parse_algo(name)
        assert ok and not ag and not auto and (s, p) == (sched, proto)
    for name in ("allgather_small", "allgather_simple", "allgather_direct", "allgather_ring:ll8"):
        ok, ag, *_ = C.parse_algo(name)
        assert ok and ag
    assert C.parse_algo("auto")[2] and C.parse_algo("nvls")[3] == "nvls" and C.parse_algo("bulk")[3] == "bulk"
    assert C.parse_algo("sequential:ll8")[3:5] == ("sequential", "LL8")
    assert not C.parse_algo("nonsense")[0] and not C.parse_algo("ring:ll7")[0]
