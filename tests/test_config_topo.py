"""Configuration tiers, HCCL_ALGO grammar, selector decisions, rank tables and topology discovery."""
import ctypes
import json

import pytest

from simutil import CMD, tool_str


def _lib():
    from hcomm_b200 import _lib
    return _lib.load()


def test_env_fields_parse_validate_and_fall_back(monkeypatch):
    lib = _lib()
    monkeypatch.setenv("HCCL_BUFFSIZE", "64")
    monkeypatch.setenv("HCCL_DETERMINISTIC", "strict")
    monkeypatch.setenv("HCCL_EXEC_TIMEOUT", "-5")          # out of range -> default
    monkeypatch.setenv("HCCL_OP_EXPANSION_MODE", "AIV")
    monkeypatch.setenv("HCCL_SOCKET_FAMILY", "AF_BOGUS")   # invalid -> default
    monkeypatch.setenv("HCCL_IF_BASE_PORT", "abc")         # malformed -> default
    lib.HcommToolReloadEnv()
    get = lambda k: tool_str(lib.HcommToolGetEnv, k.encode())[1]
    assert get("HCCL_BUFFSIZE") == "64"
    assert get("HCCL_DETERMINISTIC") == "2"
    assert get("HCCL_EXEC_TIMEOUT") == "1836"
    assert get("HCCL_OP_EXPANSION_MODE") == "3"
    assert get("HCCL_SOCKET_FAMILY") == "AF_INET"
    assert get("HCCL_IF_BASE_PORT") == "0"


def test_comm_config_layout_matches_the_c_struct():
    from hcomm_b200._lib import HcclCommConfig
    cfg = HcclCommConfig.default()
    assert ctypes.sizeof(HcclCommConfig) == 2264 or ctypes.sizeof(HcclCommConfig) % 8 == 0
    assert HcclCommConfig.hcclBufferSize.offset == 24
    assert HcclCommConfig.hcclCommName.offset == 32
    assert HcclCommConfig.hcclAlgo.offset > HcclCommConfig.hcclExecTimeOut.offset
    assert cfg.hcclBufferSize == 0xFFFFFFFF and cfg.hcclSymWinMaxMemSizePerRank == 16
    assert _lib().HcclGetCommConfigCapability() & (1 << 9)   # ALGO capability bit


def test_algo_grammar():
    lib = _lib()
    ok = lambda s: tool_str(lib.HcommToolParseAlgoConfig, s.encode())
    assert ok("level0:ring;level1:H-D_R")[0] == 0
    rc, d = ok("allreduce=level0:fullmesh;level1:ring/allgather=level0:ring/others=level0:NA")
    assert rc == 0 and "allreduce=level0:mesh" in d and "allgather=level0:ring" in d
    assert ok("level9:ring")[0] == 1
    assert ok("level0:warp")[0] == 1
    assert ok("allreduce=level0:ring/allreduce=level0:NB")[0] == 1     # configured twice
    assert ok("frobnicate=level0:ring")[0] == 1


def test_selector_decisions():
    lib = _lib()
    sel = lambda cmd, n, b, mode=0, det=0, cuda=1, nvls=1, cfg="": tool_str(lib.HcommToolSelect, CMD[cmd], n, ctypes.c_uint64(b), 4, 0, mode, det, cuda, nvls, cfg.encode())
    assert sel("allreduce", 8, 1024)[1] == "allreduce/mesh_oneshot@sm"
    assert sel("allreduce", 8, 1 << 20)[1] == "allreduce/mesh@sm"
    assert sel("allreduce", 8, 1 << 28)[1] == "allreduce/nvls@nvls"
    assert sel("allreduce", 8, 1 << 28, nvls=0)[1] == "allreduce/mesh@sm"
    assert sel("allreduce", 8, 1 << 28, det=1)[1] == "allreduce/mesh@sm"           # deterministic: fixed-order kernel
    assert sel("allreduce", 8, 1 << 20, mode=1)[1].endswith("@host")               # host expansion mode
    assert sel("allreduce", 8, 1 << 20, cfg="level0:ring")[1] == "allreduce/ring@sm-ir"
    assert sel("allreduce", 8, 1 << 20, cuda=0)[1].endswith("@host")               # simulator
    assert sel("allreduce", 8, 1 << 20, mode=5, nvls=0)[0] == 5                    # NVLS demanded but absent
    assert sel("alltoall", 8, 1 << 20, mode=5)[0] == 5                             # NVLS cannot serve all-to-all
    assert sel("allreduce", 8, 1 << 20, mode=4, cfg="level0:ring")[1] == "allreduce/ring@sm-ir"
    assert sel("allgather", 6, 4096, cfg="level0:H-D_R")[1].startswith("allgather/mesh")   # unavailable algo falls back


V1 = {"status": "completed", "version": "1.0", "server_count": "2", "server_list": [
    {"server_id": "A", "host_nic_ip": "10.0.0.1", "device": [{"device_id": "0", "device_ip": "192.168.1.8", "rank_id": "0"}, {"device_id": "1", "device_ip": "192.168.1.9", "rank_id": "1"}]},
    {"server_id": "B", "host_nic_ip": "10.0.0.2", "device": [{"device_id": "0", "device_ip": "192.168.2.8", "rank_id": "2"}, {"device_id": "1", "device_ip": "192.168.2.9", "rank_id": "3"}]}]}
V2 = {"version": "2.0", "rank_count": 2, "status": "completed", "rank_list": [
    {"rank_id": 0, "device_id": 0, "local_id": 0, "level_list": [{"net_layer": 0, "net_instance_id": "az0-rack0", "net_type": "TOPO_FILE_DESC", "net_attr": "",
                                                                    "rank_addr_list": [{"addr_type": "IPV4", "addr": "223.0.0.10", "ports": ["0/0"]}]}]},
    {"rank_id": 1, "device_id": 1, "local_id": 1, "level_list": [{"net_layer": 0, "net_instance_id": "az0-rack0", "net_type": "TOPO_FILE_DESC", "net_attr": "",
                                                                    "rank_addr_list": [{"addr_type": "IPV4", "addr": "223.0.0.28", "ports": ["0/1"]}]}]}]}


def _parse(obj, rank=0):
    lib = _lib()
    js, sm = ctypes.create_string_buffer(1 << 16), ctypes.create_string_buffer(4096)
    rc = lib.HcommToolParseRankTable(json.dumps(obj).encode() if not isinstance(obj, bytes) else obj, rank, js, len(js), sm, len(sm))
    return rc, js.value.decode(), sm.value.decode()


def test_rank_table_dialects():
    rc, js, sm = _parse(V1)
    assert rc == 0 and "SERIALISATION MISMATCH" not in sm
    out = json.loads(js)
    assert out["rank_count"] == 4 and out["rank_list"][3]["level_list"][0]["net_instance_id"] == "B"
    assert "layer 0: A(2,fabric) B(2,fabric)" in sm and "layer 1" in sm and "servers 2" in sm
    rc, js, sm = _parse(V2, rank=1)
    assert rc == 0 and json.loads(js)["rank_list"][1]["level_list"][0]["rank_addr_list"][0]["addr"] == "223.0.0.28"
    assert "rank 1/2" in sm and "layer 1" not in sm


def test_rank_table_errors_name_the_problem():
    bad = json.loads(json.dumps(V1)); bad["server_list"][1]["device"][1]["rank_id"] = "1"
    assert "appears twice" in _parse(bad)[2]
    bad = json.loads(json.dumps(V1)); bad["server_count"] = "3"
    assert "server_count" in _parse(bad)[2]
    bad = json.loads(json.dumps(V2)); del bad["rank_list"][0]["device_id"]
    assert "device_id" in _parse(bad)[2]
    bad = json.loads(json.dumps(V2)); bad["rank_count"] = 5
    assert "rank_count" in _parse(bad)[2]
    assert "not valid JSON" in _parse(b"{ nope")[2]
    bad = json.loads(json.dumps(V2)); bad["status"] = "initializing"
    assert "status" in _parse(bad)[2]


def test_generated_topologies_and_links():
    lib = _lib()
    js, sm = ctypes.create_string_buffer(1 << 20), ctypes.create_string_buffer(4096)
    assert lib.HcommToolGenTopo(1, 1, 8, 3, js, len(js), sm, len(sm)) == 0
    assert "pod0-srv0(8,fabric)" in sm.value.decode() and "L0 link to next: 1 proto 16 hop 2" in sm.value.decode()
    assert lib.HcommToolGenTopo(2, 2, 4, 3, js, len(js), sm, len(sm)) == 0
    s = sm.value.decode()
    # rank 3 and rank 4 sit on different hosts: no layer-0 link, one RoCE link at layer 1
    assert "L0 link to next: 0" in s and "L1 link to next: 1 proto 1 hop 3" in s and "layer 2" in s


def test_nvml_discovery_through_a_fake_table():
    lib = _lib()
    rc, s = tool_str(lib.HcommToolFakeNvmlProbe, 8, 1)
    assert rc == 0 and s.startswith("gpus 8") and "links 18 switch 18 peers 0 fabric 1" in s
    rc, s = tool_str(lib.HcommToolFakeNvmlProbe, 2, 0)
    assert rc == 0 and "links 18 switch 0 peers 18 fabric 0" in s
    tool_str(lib.HcommToolFakeNvmlProbe, 0, 0)


def test_parsers_survive_damaged_input():
    """tests/fuzz_parsers.py: a few thousand rank tables and algorithm settings with values replaced, removed, duplicated,
    bytes flipped, cut and nested far too deep.  Every one is answered with a return code; what is accepted parses again."""
    import subprocess
    import sys
    from pathlib import Path
    run = subprocess.run([sys.executable, str(Path(__file__).resolve().parent / "fuzz_parsers.py"), "2500", "11"], capture_output=True, text=True, errors="replace", timeout=600)
    assert run.returncode == 0 and "fuzz: 2500 inputs" in run.stdout, run.stdout[-2000:] + run.stderr[-4000:]
    rc, _, sm = _parse(b'{"a":' + b"[" * 200000 + b"]" * 200000 + b"}")
    assert rc != 0 and "nesting too deep" in sm


def test_communicator_creation_survives_damaged_configuration_structures():
    import subprocess
    import sys
    from pathlib import Path
    run = subprocess.run([sys.executable, str(Path(__file__).resolve().parent / "fuzz_config.py"), "120", "3"], capture_output=True, text=True, errors="replace", timeout=600)
    assert run.returncode == 0 and "config fuzz: 120 structures" in run.stdout, run.stdout[-2000:] + run.stderr[-4000:]
