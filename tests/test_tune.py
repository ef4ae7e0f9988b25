"""The tuner's table construction and the selector's use of a tuning file."""
import ctypes
import json
import os

from hcomm_b200.utils.tune import merge_buckets, pick_winners


def test_winners_are_sticky_and_buckets_merge():
    meas = {
        1024: {("mesh_oneshot", "sm", 0): 10.0, ("mesh", "sm", 0): 14.0},
        4096: {("mesh_oneshot", "sm", 0): 11.0, ("mesh", "sm", 0): 10.9},         # within 3 %: the incumbent stays
        1 << 20: {("mesh_oneshot", "sm", 0): 60.0, ("mesh", "sm", 0): 30.0, ("nvls", "nvls", 64): 40.0},
        1 << 24: {("mesh", "sm", 0): 200.0, ("nvls", "nvls", 64): 120.0},
    }
    winners = pick_winners(meas)
    assert [w[1] for w in winners] == ["mesh_oneshot", "mesh_oneshot", "mesh", "nvls"]
    buckets = merge_buckets(winners)
    assert buckets == [{"max_bytes": 4096, "algo": "mesh_oneshot", "engine": "sm", "ctas": 0},
                       {"max_bytes": 1 << 20, "algo": "mesh", "engine": "sm", "ctas": 0},
                       {"max_bytes": -1, "algo": "nvls", "engine": "nvls", "ctas": 64}]


def test_selector_follows_a_tuning_file(tmp_path, monkeypatch):
    from hcomm_b200 import _lib
    lib = _lib.load()
    table = {"allreduce": {"8": [{"max_bytes": 2048, "algo": "mesh_oneshot", "engine": "sm", "ctas": 2},
                                 {"max_bytes": -1, "algo": "mesh", "engine": "sm", "ctas": 96}]}}
    path = tmp_path / "tune.json"
    path.write_text(json.dumps(table))
    monkeypatch.setenv("HCCL_TUNE_FILE", str(path))
    lib.HcommToolReloadEnv()
    try:
        out = ctypes.create_string_buffer(512)
        # cmd 2 = all-reduce, 8 ranks, bf16 (11) sum (0), default expansion mode, not deterministic, on CUDA with NVLS
        assert lib.HcommToolSelect(2, 8, ctypes.c_uint64(1024), 11, 0, 0, 0, 1, 1, b"", out, 512) == 0
        assert "mesh_oneshot" in out.value.decode()
        assert lib.HcommToolSelect(2, 8, ctypes.c_uint64(1 << 26), 11, 0, 0, 0, 1, 1, b"", out, 512) == 0
        text = out.value.decode()
        assert "mesh" in text and "oneshot" not in text and "nvls" not in text, text
    finally:
        monkeypatch.delenv("HCCL_TUNE_FILE")
        lib.HcommToolReloadEnv()


def test_table_from_sweep_files_counts_bytes_like_the_selector(tmp_path):
    from hcomm_b200.utils.tune import table_from_sweeps
    mesh = [{"op": "allgather", "bytes": b, "n": 8, "algo": "auto", "ours_us": t} for b, t in ((1 << 20, 25.0), (1 << 22, 54.0), (1 << 24, 72.0), (1 << 26, 143.0))]
    nvls = [{"op": "allgather", "bytes": b, "n": 8, "algo": "allgather=level0:nvls/reducescatter=level0:nvls", "ours_us": t}
            for b, t in ((1 << 20, 35.0), (1 << 22, 39.0), (1 << 24, 57.0), (1 << 26, 152.0))]
    a, b = tmp_path / "mesh.json", tmp_path / "nvls.json"
    a.write_text(json.dumps(mesh))
    b.write_text(json.dumps(nvls))
    table = table_from_sweeps([str(a), str(b)], ["allgather"], "mesh")
    # sizes are per rank (what the selector compares): 128 KB, 512 KB, 2 MB, 8 MB
    assert table == {"allgather": {"8": [{"max_bytes": 1 << 17, "algo": "mesh", "engine": "sm", "ctas": 0},
                                         {"max_bytes": 1 << 21, "algo": "nvls", "engine": "nvls", "ctas": 0},
                                         {"max_bytes": -1, "algo": "mesh", "engine": "sm", "ctas": 0}]}}


def test_built_in_all_gather_buckets_match_the_shipped_table():
    from pathlib import Path
    from hcomm_b200 import _lib
    import hcomm_b200.utils.tune as tune
    lib = _lib.load()
    shipped = json.loads((Path(tune.__file__).parent / "tune_tables" / "b200_8gpu_allgather_reducescatter.json").read_text())
    out = ctypes.create_string_buffer(512)
    edges = [0] + [b["max_bytes"] for b in shipped["allgather"]["8"][:-1]]
    for bucket, lo in zip(shipped["allgather"]["8"], edges):
        size = lo + 4096 if bucket["max_bytes"] < 0 else bucket["max_bytes"]
        # cmd 6 = all-gather, 8 ranks, bf16, on CUDA with NVLS available
        assert lib.HcommToolSelect(6, 8, ctypes.c_uint64(size), 11, 0, 0, 0, 1, 1, b"", out, 512) == 0
        assert ("nvls" in out.value.decode()) == (bucket["algo"] == "nvls"), (size, out.value.decode())
