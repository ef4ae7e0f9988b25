"""Creates one-rank communicators from configuration structures with damaged bytes (``fuzz_config.py <iterations> <seed>``).
Every structure is either refused with a return code or gives a communicator that can be destroyed; the process survives.
Run as a child process by the tests, also on the AddressSanitizer build."""
import ctypes
import os
import random
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
os.environ.setdefault("HCCL_SIM", "1")


def main():
    iterations, seed = int(sys.argv[1]), int(sys.argv[2])
    import hcomm_b200 as hb
    from hcomm_b200 import _lib
    lib = _lib.load()
    rng = random.Random(seed)
    size = ctypes.sizeof(_lib.HcclCommConfig)
    accepted = refused = 0
    for _ in range(iterations):
        info = _lib.HcclRootInfo()
        raw = hb.get_root_info()
        ctypes.memmove(ctypes.addressof(info), raw, len(raw))
        cfg = _lib.HcclCommConfig.default()
        view = (ctypes.c_ubyte * size).from_address(ctypes.addressof(cfg))
        for _ in range(rng.randint(1, 12)):                   # a few bytes behind the 24-byte header
            view[rng.randrange(24, size)] = rng.randrange(256)
        if rng.random() < 0.7:
            cfg.hcclBufferSize = rng.choice([1, 2, 0xffffffff])   # small or "not set": memory is not what is tested here
        if rng.random() < 0.1:
            view[rng.randrange(0, 24)] = rng.randrange(256)   # now and then the header itself
        handle = ctypes.c_void_p()
        rc = lib.HcclCommInitRootInfoConfig(1, ctypes.byref(info), 0, ctypes.byref(cfg), ctypes.byref(handle))
        if rc == 0:
            accepted += 1
            assert lib.HcclCommDestroy(handle) == 0
        else:
            refused += 1
    print(f"config fuzz: {iterations} structures, {accepted} accepted, {refused} refused", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
