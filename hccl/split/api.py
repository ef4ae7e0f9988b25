"""Gradient-fusion split strategy (``HcomSetGradFusionByIndex`` / ``BySize``).

A strategy cuts the list of gradients of a model into at most 8 contiguous segments; every segment is
all-reduced as one fused buffer as soon as its last gradient is ready, so communication of early
segments overlaps the rest of the backward pass.
"""
import ctypes

from ..manage.api import WORLD_GROUP, _lib, check_group

MAX_SEGMENTS = 8


def set_split_strategy_by_idx(idxList, group=WORLD_GROUP):
    """``idxList``: ascending indices of the last gradient of each segment."""
    check_group(group)
    if not isinstance(idxList, list):
        raise ValueError("idxList must be a python list")
    if len(idxList) == 0 or len(idxList) > MAX_SEGMENTS:
        raise ValueError(f"idxList length must be in [1, {MAX_SEGMENTS}]")
    last = -1
    for v in idxList:
        if not isinstance(v, int) or isinstance(v, bool) or v < 0:
            raise ValueError("idxList values must be non-negative python ints")
        if v <= last:
            raise ValueError("idxList must be strictly ascending")
        last = v
    arr = (ctypes.c_uint * len(idxList))(*idxList)
    ret = _lib().HcomSetGradFusionByIndex(group.encode("utf-8"), ctypes.c_uint(len(idxList)), arr)
    if ret != 0:
        raise ValueError(f"set split strategy by idx error. ret[{ret}]")


def set_split_strategy_by_size(dataSizeList, group=WORLD_GROUP):
    """``dataSizeList``: percentage of the total gradient bytes per segment; must sum to 100."""
    check_group(group)
    if not isinstance(dataSizeList, list):
        raise ValueError("dataSizeList must be a python list")
    if len(dataSizeList) == 0 or len(dataSizeList) > MAX_SEGMENTS:
        raise ValueError(f"dataSizeList length must be in [1, {MAX_SEGMENTS}]")
    total = 0.0
    for v in dataSizeList:
        if not isinstance(v, (int, float)) or isinstance(v, bool) or v < 0:
            raise ValueError("dataSizeList values must be non-negative numbers")
        total += float(v)
    if abs(total - 100.0) > 1e-3:
        raise ValueError(f"dataSizeList must sum to 100, got {total}")
    arr = (ctypes.c_float * len(dataSizeList))(*[float(v) for v in dataSizeList])
    ret = _lib().HcomSetGradFusionBySize(group.encode("utf-8"), ctypes.c_uint(len(dataSizeList)), arr)
    if ret != 0:
        raise ValueError(f"set split strategy by size error. ret[{ret}]")


def get_split_strategy(grad_bytes, group=WORLD_GROUP):
    """Resolves the stored strategy for gradients of the given byte sizes into segment end indices."""
    check_group(group)
    n = len(grad_bytes)
    sizes = (ctypes.c_uint64 * n)(*[int(b) for b in grad_bytes])
    seg = (ctypes.c_uint * n)()
    cnt = ctypes.c_uint()
    ret = _lib().HcomGetSplitStrategy(group.encode("utf-8"), ctypes.c_uint(n), sizes, seg, ctypes.byref(cnt))
    if ret != 0:
        raise ValueError(f"get split strategy error. ret[{ret}]")
    return [seg[i] for i in range(cnt.value)]
