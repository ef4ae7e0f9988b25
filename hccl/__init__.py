"""Python ``hccl`` package: group management and gradient-split strategy on top of ``libhcomm.so``.

API parity with the reference's ``python/hccl`` (``hccl.manage.api``, ``hccl.split.api``).  The
world group must exist first: a process joins it with :func:`hccl.manage.api.init_world_group`
(root-info bootstrap, or adopting an existing communicator handle) or, as in the reference,
through a rank table (``HcomInitByRankTable``).
"""
