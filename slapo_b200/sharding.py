"""Sharding API under the reference's package name ``sharding``."""
from .parallel.reshard_ops import *  # noqa: F401,F403
from .parallel.reshard_ops import parse_reshard, reshard  # noqa: F401
from .parallel.shard_methods import (SHARD_METHODS, ShardMethod, SyncFn, SyncHook,  # noqa: F401
                                     apply_shard_method, apply_sync_method,
                                     new_or_get_tied_param, register_shard_method)
from .parallel.sync_ops import (all_gather_along_dim, all_gather_forward_output,  # noqa: F401
                                reduce_backward_grad, reduce_forward_output,
                                reduce_scatter_along_dim, reduce_scatter_forward_output,
                                scatter_along_dim, scatter_forward_output)
