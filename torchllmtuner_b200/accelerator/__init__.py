"""L1 accelerator runtime: device selection, process-group bring-up, collective services, capability probes."""
from .capabilities import has, report, require  # noqa: F401
from .collectives import (CoordinatedError, PartialToInvariantAllReduce, agree_status, all_reduce, set_pg_timeouts,  # noqa: F401
                          synchronize_after_wait, synchronize_local_errors)
from .device import (get_current_device, get_device_type, get_distributed_backend, get_env_dist_info, set_device,  # noqa: F401
                     should_use_pin_memory)
from .distributed import (barrier, destroy, get_comm_device, get_dist_info, get_rank, get_world_size, infer_launcher,  # noqa: F401
                          init_dist, init_dist_pytorch, is_distributed, is_main_process, master_only)
from .tensor_tree import get_tensor_tree_device, move_tensor_tree  # noqa: F401
