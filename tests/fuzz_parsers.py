"""Feeds damaged rank tables and algorithm settings to the parsers of the library.  Run as a script (the tests start it as a
child process, also on the AddressSanitizer build): ``fuzz_parsers.py <iterations> <seed>``.  Every input must come back
with a return code and a message; the process must survive."""
import ctypes
import json
import random
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

V1 = {"status": "completed", "version": "1.0", "server_count": "2", "server_list": [
    {"server_id": "A", "host_nic_ip": "10.0.0.1", "device": [{"device_id": "0", "device_ip": "192.168.1.8", "rank_id": "0"}, {"device_id": "1", "device_ip": "192.168.1.9", "rank_id": "1"}]},
    {"server_id": "B", "host_nic_ip": "10.0.0.2", "device": [{"device_id": "0", "device_ip": "192.168.2.8", "rank_id": "2"}, {"device_id": "1", "device_ip": "192.168.2.9", "rank_id": "3"}]}]}
V2 = {"version": "2.0", "rank_count": 2, "status": "completed", "rank_list": [
    {"rank_id": 0, "device_id": 0, "local_id": 0, "level_list": [{"net_layer": 0, "net_instance_id": "az0-rack0", "net_type": "TOPO_FILE_DESC", "net_attr": "",
                                                                    "rank_addr_list": [{"addr_type": "IPV4", "addr": "223.0.0.10", "ports": ["0/0"]}]}]},
    {"rank_id": 1, "device_id": 1, "local_id": 1, "level_list": [{"net_layer": 0, "net_instance_id": "az0-rack0", "net_type": "TOPO_FILE_DESC", "net_attr": "",
                                                                    "rank_addr_list": [{"addr_type": "IPV4", "addr": "223.0.0.28", "ports": ["0/1"]}]}]}]}
ALGOS = ["level0:ring", "level0:H-D_R;level1:NHR", "allreduce=level0:fullmesh;level1:ring/allgather=level0:NB", "level0:pairwise", "level3:NA",
         "alltoall=level0:pairwise;level1:pairwise/others=level0:ring"]
ODD = [None, True, False, -1, 0, 1 << 40, 1e308, "", "x" * 3000, [], {}, [[[]]], {"a": {"a": {"a": {}}}}, "\u0000", "9" * 40, "-", "0x10", " 7 "]


def odd(rng):
    return json.loads(json.dumps(rng.choice(ODD)))        # a copy: the lists and dicts among them get changed later


def damaged_object(rng, obj):
    """A copy of obj with a few values replaced, removed or duplicated at random places."""
    obj = json.loads(json.dumps(obj))
    for _ in range(rng.randint(1, 4)):
        node, steps = obj, 0
        while steps < 8:
            steps += 1
            if isinstance(node, dict) and node:
                key = rng.choice(list(node))
                if isinstance(node[key], (dict, list)) and node[key] and rng.random() < 0.7:
                    node = node[key]
                    continue
                act = rng.random()
                if act < 0.4:
                    node[key] = odd(rng)
                elif act < 0.7:
                    del node[key]
                else:
                    node[key + rng.choice(["", "_", "2"])] = odd(rng)
                break
            if isinstance(node, list) and node:
                i = rng.randrange(len(node))
                if isinstance(node[i], (dict, list)) and node[i] and rng.random() < 0.7:
                    node = node[i]
                    continue
                act = rng.random()
                if act < 0.3:
                    node[i] = odd(rng)
                elif act < 0.6:
                    del node[i]
                else:
                    node.extend(json.loads(json.dumps(node)) * rng.randint(1, 3))
                break
            break
    return obj


def damaged_bytes(rng, data):
    data = bytearray(data)
    for _ in range(rng.randint(1, 6)):
        if not data:
            break
        act, i = rng.random(), rng.randrange(len(data))
        if act < 0.3:
            data[i] = rng.randrange(256)
        elif act < 0.5:
            del data[i:i + rng.randint(1, 30)]
        elif act < 0.7:
            data[i:i] = bytes(rng.choice(b'{}[]",:\\-0123456789eE.tfn ') for _ in range(rng.randint(1, 20)))
        elif act < 0.85:
            data = data[:i]
        else:
            data[i:i] = b"[" * rng.randint(50, 3000)      # nesting far beyond any table
    return bytes(data)


def main():
    iterations, seed = int(sys.argv[1]), int(sys.argv[2])
    from hcomm_b200 import _lib
    lib = _lib.load()
    rng = random.Random(seed)
    js, sm, out = ctypes.create_string_buffer(1 << 18), ctypes.create_string_buffer(4096), ctypes.create_string_buffer(1 << 14)
    accepted = refused = 0
    for it in range(iterations):
        base = rng.choice((V1, V2))
        text = json.dumps(damaged_object(rng, base)).encode()
        if rng.random() < 0.5:
            text = damaged_bytes(rng, text)
        text = text.replace(b"\x00", b" ")                # the entry point takes a C string
        rc = lib.HcommToolParseRankTable(text, rng.randrange(6), js, len(js), sm, len(sm))
        if rc == 0:
            accepted += 1
            json.loads(js.value.decode(errors="replace"))                 # what it accepted comes back as a table that parses
        else:
            refused += 1
            assert sm.value, "a refusal without a message"
        algo = rng.choice(ALGOS).encode()
        if rng.random() < 0.8:
            algo = damaged_bytes(rng, algo).replace(b"\x00", b" ")[:4000]
        lib.HcommToolParseAlgoConfig(algo, out, len(out))
    print(f"fuzz: {iterations} inputs, {accepted} accepted, {refused} refused", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
