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
