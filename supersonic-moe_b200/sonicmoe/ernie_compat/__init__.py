from .deepep_metadata import deepep_topk_to_sonic_metadata, metadata_lanes_expert_sorted  # noqa: F401
