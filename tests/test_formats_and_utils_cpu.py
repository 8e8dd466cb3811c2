"""Properties of the wire formats (through the emulator's image builder) and of the bandwidth helpers."""
import numpy as np
import pytest

import emu
from gpu_ipc_example_b200 import utils

SPEC = {"LL8": (64, 32), "LL16": (128, 64), "LL128": (32, 30), "LL512": (128, 120)}


@pytest.mark.parametrize("proto", list(SPEC))
def test_every_payload_dword_has_its_own_slot_and_the_rest_are_flags(proto):
    txn_dw, payload_dw = SPEC[proto]
    L = emu.lib()
    assert L.b200emu_payload_dw(emu.PROTOS[proto]) == payload_dw
    assert L.b200emu_txn_bytes(emu.PROTOS[proto]) == txn_dw * 4
    flag = 0xFFFFFFFF
    payload = np.arange(1, payload_dw + 1, dtype=np.uint32)
    img = emu.wire_image(proto, payload, flag)
    assert len(img) == txn_dw
    data_slots = [i for i, v in enumerate(img) if v != flag]
    assert sorted(int(img[i]) for i in data_slots) == list(range(1, payload_dw + 1))  # a bijection onto the non-flag slots
    assert len(data_slots) == payload_dw and txn_dw - payload_dw == int((img == flag).sum())


@pytest.mark.parametrize("proto,unit_bytes", [("LL8", 8), ("LL16", 8), ("LL128", 64), ("LL512", 64)])
def test_every_atomic_unit_carries_a_flag(proto, unit_bytes):
    """The protocols rely on payload and flag sharing one atomic unit: 8-byte granules for LL8/LL16,
    64-byte segments for LL128/LL512 (rt64_128.hpp:544: a 128-byte transaction is not atomic)."""
    flag = 0xFFFFFFFF
    img = emu.wire_image(proto, np.zeros(SPEC[proto][1], np.uint32), flag)
    per_unit = unit_bytes // 4
    for u in range(len(img) // per_unit):
        unit = img[u * per_unit:(u + 1) * per_unit]
        assert (unit == flag).any()
        assert unit[-1] == flag  # the flag closes the unit


def test_payload_efficiency_matches_the_reference_formats():
    eff = {p: SPEC[p][1] / SPEC[p][0] for p in SPEC}
    assert eff["LL8"] == eff["LL16"] == 0.5            # rt64.hpp:339-340, 8-9
    assert eff["LL128"] == eff["LL512"] == 0.9375      # rt64_128.hpp:549-550, 7-10


def test_bandwidth_conventions():
    assert utils.allreduce_busbw_gbs(16 << 20, 60e-6, 8) == pytest.approx((16 << 20) / 60e-6 / 1e9 * 1.75)
    assert utils.allgather_busbw_gbs(8 << 20, 1e-4, 8) == pytest.approx((8 << 20) / 1e-4 / 1e9 * 0.875)
    assert utils.allreduce_link_bound_gbs(8, nvls=False) == 770.0
    assert utils.allreduce_link_bound_gbs(8, nvls=True) == pytest.approx(770.0 * 14 / 9)
    p = utils.load_peaks("/nonexistent")
    assert p.source == "fallback" and p.bf16_tflops == 1590.0
    # M = 2048 at TP = 8: at the nominal 900 GB/s the GEMM at the measured peak is the slower side, at the
    # measured 770 GB/s peer-copy rate the link is; M = 1 is (nominally) compute bound at a sliver of a microsecond
    big = utils.fused_layer_roofline_seconds(2048, 3584, 8192, 8, p)
    assert big == pytest.approx(max(2 * 7 / 8 * 2048 * 8192 * 2 / 900e9, 2 * 2048 * 3584 * 8192 / 1590e12))
    assert utils.fused_layer_roofline_seconds(2048, 3584, 8192, 8, p, utils.NVLINK_PEER_COPY_GBS) == pytest.approx(2 * 7 / 8 * 2048 * 8192 * 2 / 770e9)
    assert utils.fused_layer_roofline_seconds(1, 3584, 8192, 1, p) == pytest.approx(2 * 3584 * 8192 / 1590e12)


def test_tuner_picks_the_fastest_algorithm_per_size():
    from gpu_ipc_example_b200 import tune

    a = tune.parse_sweep("# world 8\n#  elements bytes ctas warps time_us(max) algbw busbw\n"
                         "  1024 2048 1 8 10.00 0.2 0.4\n  1048576 2097152 64 16 60.00 30.0 60.0\n")
    b = tune.parse_sweep("  1024 2048 1 8 12.00 0.2 0.3\n  1048576 2097152 64 16 23.00 90.0 150.0\n  4194304 8388608 64 16 40.0 200 350\n")
    assert a == {1024: 10.0, 1048576: 60.0}
    rows = tune.best_per_size({"oneshot:ll512": a, "parallel:ll512": b})
    assert [(r[0], r[1]) for r in rows] == [(1024, "oneshot:ll512"), (1048576, "parallel:ll512"), (4194304, "parallel:ll512")]
    merged = tune.merge_rows(rows)
    assert merged == [(2048, "oneshot:ll512"), (0, "parallel:ll512")]
    cpp = tune.as_cpp(merged)
    assert "{2 * KiB, SchedKind::OneShot, ProtoKind::LL512}," in cpp and "{0, SchedKind::Parallel, ProtoKind::LL512}," in cpp


def test_tuner_reads_json_rows_and_limits_the_row_count():
    import json

    from gpu_ipc_example_b200 import tune

    nine = tune.parse_sweep("  1024 2048 1 8 9.00 10.00 12.00 0.2 0.4\n")
    assert nine == {1024: 10.0}  # the median column of the nine-column table
    rows = []
    times = {"oneshot:ll512": [5, 6, 9, 30, 90, 300], "parallel:ll512": [8, 8, 8.5, 12, 40, 150], "bisect:ll512": [9, 9, 9, 11.9, 41, 151],
             "nvls": [17, 17, 17, 18, 25, 60]}
    for algo, ts in times.items():
        for e, us in zip((10, 12, 14, 16, 18, 20), ts):
            rows.append(json.dumps({"collective": "all_reduce", "algo": algo, "world": 8, "placement": "in_place", "symmetric": False,
                                    "elements": 1 << e, "us_median": us}))
    rows.append(json.dumps({"collective": "all_reduce", "algo": "nvls", "world": 4, "placement": "in_place", "symmetric": False,
                            "elements": 1024, "us_median": 1.0}))
    tables = tune.parse_json_rows("\n".join(rows), 8)
    assert set(tables) == set(times) and tables["nvls"][1024] == 17
    every = tune.merge_rows(tune.best_per_size(tables))
    assert [a for _, a in every] == ["oneshot:ll512", "parallel:ll512", "bisect:ll512", "nvls"]
    three = tune.best_table(tables, 3)
    assert three == [(2 << 12, "oneshot:ll512"), (2 << 16, "parallel:ll512"), (0, "nvls")]


def test_tuner_cut_offs_for_all_gather_and_reduce_scatter(tmp_path, capsys, monkeypatch):
    """`--collective`: the same rows give the cut-offs of the other two collectives (NCCL rows are shown, never picked)."""
    import json
    import sys

    from gpu_ipc_example_b200 import tune

    rows = []
    times = {"allgather_direct": [5, 6, 30, 90], "allgather_bulk": [12, 12, 20, 70], "allgather_simple": [9, 9, 25, 50],
             "nccl_allgather": [4, 4, 4, 4], "allgather_auto": [1, 1, 1, 1]}
    for algo, ts in times.items():
        for e, us in zip((10, 14, 18, 22), ts):
            rows.append(json.dumps({"collective": "all_gather", "algo": algo, "world": 8, "placement": "out_of_place", "symmetric": False,
                                    "elements": 1 << e, "us_median": us}))
    path = tmp_path / "rows.jsonl"
    path.write_text("\n".join(rows) + "\n")
    monkeypatch.setattr(sys, "argv", ["tune", "--from-json", str(path), "--np", "8", "--collective", "all_gather", "--max-rows", "3"])
    tune.main()
    out = capsys.readouterr().out
    assert "nccl" not in out.split("up to", 1)[1] and "allgather_auto" not in out
    cut = [line.split(": ")[1] for line in out.splitlines() if line.startswith("up to")]
    assert cut == ["allgather_direct", "allgather_bulk", "allgather_simple"]
    assert "(4.0)" in out  # the NCCL time beside every winner
