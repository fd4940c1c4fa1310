from .state import (
    GroupCoordinator, data_parallel_all_reduce, destroy_model_parallel, get_dp_group, get_ep_group,
    get_pp_group, get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size, get_tp_group,
    init_distributed, initialize_model_parallel, model_parallel_is_initialized,
    tensor_model_parallel_all_gather, tensor_model_parallel_all_reduce,
)
