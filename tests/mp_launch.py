"""Starts `world` copies of mp_worker.py and collects their exit codes."""
import os
import subprocess
import sys
import tempfile
from pathlib import Path

WORKER = str(Path(__file__).resolve().parent / "mp_worker.py")


def launch(scenario, world, env_extra=None, timeout=180):
    with tempfile.TemporaryDirectory() as tmp:
        procs = []
        for r in range(world):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), HCOMM_ROOT_FILE=str(Path(tmp) / "root.bin"))
            env.update(env_extra or {})
            procs.append(subprocess.Popen([sys.executable, WORKER, scenario], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, errors="replace"))
        codes, outs = [], []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=timeout)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
                out += "\n<killed after timeout>"
            codes.append(p.returncode)
            outs.append(out)
        return codes, outs
