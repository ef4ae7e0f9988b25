"""Group management: create / destroy named groups and translate ranks (``Hcom*`` C API)."""
import ctypes

MAX_GROUP_NAME_LEN = 127
WORLD_GROUP = "hccl_world_group"


def _lib():
    from hcomm_b200 import _lib as binding
    return binding.load()


def check_group(group):
    if not isinstance(group, str):
        raise ValueError("group must be a python str")
    if len(group) == 0:
        raise ValueError("group name is empty.")
    if len(group) > MAX_GROUP_NAME_LEN:
        raise ValueError("group name is invalid. group: " + group[:MAX_GROUP_NAME_LEN])


def check_rank_num(rank_num):
    if not isinstance(rank_num, int) or isinstance(rank_num, bool):
        raise ValueError("rank_num must be a python int")
    if rank_num <= 0:
        raise ValueError(f"rank_num[{rank_num}] is less than 0 or equal to 0")


def check_rank_id(rank_id):
    if not isinstance(rank_id, int) or isinstance(rank_id, bool):
        raise ValueError("rank_id must be a python int")
    if rank_id < 0:
        raise ValueError(f"rank_id[{rank_id}] is less than 0")


def init_world_group(comm_handle):
    """Adopts an existing communicator (``Communicator.handle``) as ``hccl_world_group``."""
    ret = _lib().HcomInitByComm(ctypes.c_void_p(comm_handle))
    if ret != 0:
        raise ValueError(f"init world group error. ret[{ret}]")


def init_world_group_by_rank_table(rank_table_path, rank_id):
    check_rank_id(rank_id)
    ret = _lib().HcomInitByRankTable(rank_table_path.encode("utf-8"), ctypes.c_uint(rank_id))
    if ret != 0:
        raise ValueError(f"init by rank table error. ret[{ret}]")


def destroy_world_group():
    _lib().HcomDestroy()


def create_group(group, rank_num, rank_ids):
    check_group(group)
    check_rank_num(rank_num)
    if not isinstance(rank_ids, list):
        raise ValueError("rank_ids must be a python list")
    if rank_num != len(rank_ids):
        raise ValueError(f"rank_num[{rank_num}] not equal to rank_ids len[{len(rank_ids)}].")
    for r in rank_ids:
        check_rank_id(r)
    arr = (ctypes.c_uint * len(rank_ids))(*rank_ids)
    ret = _lib().HcomCreateGroup(group.encode("utf-8"), ctypes.c_uint(rank_num), arr)
    if ret != 0:
        raise ValueError("create group error:" + group)


def destroy_group(group):
    check_group(group)
    ret = _lib().HcomDestroyGroup(group.encode("utf-8"))
    if ret != 0:
        raise ValueError("destroy group error :" + group)


def _query(fn_name, group, what):
    check_group(group)
    out = ctypes.c_uint()
    ret = getattr(_lib(), fn_name)(group.encode("utf-8"), ctypes.byref(out))
    if ret != 0:
        raise ValueError(f"get {what} error. ret[{ret}]")
    return out.value


def get_rank_size(group=WORLD_GROUP):
    return _query("HcomGetRankSize", group, "rank size")


def get_rank_id(group=WORLD_GROUP):
    return _query("HcomGetRankId", group, "rank id")


def get_local_rank_size(group=WORLD_GROUP):
    return _query("HcomGetLocalRankSize", group, "local rank size")


def get_local_rank_id(group=WORLD_GROUP):
    return _query("HcomGetLocalRankId", group, "local rank id")


def get_world_rank_from_group_rank(group, group_rank_id):
    check_group(group)
    check_rank_id(group_rank_id)
    out = ctypes.c_uint()
    ret = _lib().HcomGetWorldRankFromGroupRank(group.encode("utf-8"), ctypes.c_uint(group_rank_id), ctypes.byref(out))
    if ret != 0:
        raise ValueError(f"get world rank from group rank error. ret[{ret}]")
    return out.value


def get_group_rank_from_world_rank(world_rank_id, group):
    check_group(group)
    check_rank_id(world_rank_id)
    out = ctypes.c_uint()
    ret = _lib().HcomGetGroupRankFromWorldRank(ctypes.c_uint(world_rank_id), group.encode("utf-8"), ctypes.byref(out))
    if ret != 0:
        raise ValueError(f"get group rank from world rank error. ret[{ret}]")
    return out.value
