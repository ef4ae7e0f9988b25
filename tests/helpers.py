"""Shared helpers: run one function per rank in threads of this process."""
import threading
import time
import traceback


def run_ranks(n, fn, timeout=120):
    """Calls fn(rank) in n threads; re-raises the first failure; returns the per-rank results."""
    results, errors = [None] * n, []

    def wrap(r):
        try:
            results[r] = fn(r)
        except BaseException as e:  # noqa: BLE001
            errors.append((r, e, traceback.format_exc()))

    threads = [threading.Thread(target=wrap, args=(r,), daemon=True) for r in range(n)]
    for t in threads:
        t.start()
    # Wait for all ranks, but once one has failed give the others only a short grace period: they are usually
    # blocked in a collective the failed rank will never join, and the first failure is the one worth reporting.
    deadline = time.time() + timeout
    failed_at = None
    while any(t.is_alive() for t in threads) and time.time() < deadline:
        if errors and failed_at is None:
            failed_at = time.time()
        if failed_at is not None and time.time() - failed_at > 3.0:
            break
        time.sleep(0.005)
    if errors:
        r, e, tb = errors[0]
        raise AssertionError(f"rank {r} failed: {e}\n{tb}")
    if any(t.is_alive() for t in threads):
        raise TimeoutError("a rank thread did not finish")
    return results
