from .api import (create_group, destroy_group, get_group_rank_from_world_rank, get_local_rank_id, get_local_rank_size,  # noqa: F401
                  get_rank_id, get_rank_size, get_world_rank_from_group_rank, init_world_group, init_world_group_by_rank_table,
                  destroy_world_group)
