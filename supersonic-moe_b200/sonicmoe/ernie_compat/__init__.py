from .deepep_metadata import (deepep_topk_to_sonic_metadata, deepep_topk_to_sonic_metadata_with_scales,  # noqa: F401
                              metadata_lanes_expert_sorted)
from .mlp_node_v2 import SonicMoEMlpNode, flush_w1_main_grad_, stack_w1_interleaved, stack_w2  # noqa: F401,E402
