"""Shared helpers: run one function per rank in threads of this process."""
import threading
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
    for t in threads:
        t.join(timeout)
        if t.is_alive():
            raise TimeoutError("a rank thread did not finish")
    if errors:
        r, e, tb = errors[0]
        raise AssertionError(f"rank {r} failed: {e}\n{tb}")
    return results
