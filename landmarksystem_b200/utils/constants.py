"""Key names shared by the inference configuration, the engine and the offload stack."""

_RANK_STR, _WORLD_SIZE_STR = "rank", "world_size"                                   # filled into ``parallel_config``
_PARALLEL_CONFIG_STR, _OFFLOAD_CONFIG_STR = "parallel_config", "offload_config"     # sections of the inference configuration
MERGE_TYPE_STR = "merge_type"                                                       # key of a component's merge description
