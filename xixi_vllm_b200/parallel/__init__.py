"""Distributed layer: process groups, collectives, control channel, pipeline helpers."""

from .collectives import (all_gather, all_reduce, recv_tensors, reduce_scatter, send_tensors,
                          tensor_model_parallel_all_gather, tensor_model_parallel_all_reduce,
                          tensor_model_parallel_reduce_scatter)
from .control_channel import ControlChannel
from .groups import (Group, destroy_distributed_environment, destroy_model_parallel, get_pp_group,
                     get_tp_group, get_world_group, graph_capture, init_distributed_environment,
                     initialize_model_parallel, model_parallel_is_initialized, set_nccl_env,
                     single_process_groups)
from .pp import IntermediateTensors, PPMissingLayer, divide, get_pp_indices, set_pp_layer_ranges

__all__ = [n for n in dir() if not n.startswith("_")]
