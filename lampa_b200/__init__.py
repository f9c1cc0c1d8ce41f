"""lampa_b200: B200 (sm_100a) implementation of Lampa's LSH ordering and (hierarchical)
chunkwise gated-delta-rule forward, behind the reference's own Python entry points."""
from ._lib import LampaError, check_status  # noqa: F401
from .gated_delta import (  # noqa: F401
    HState, HStruct, HType, chunk_gated_delta_rule, chunk_h_gated_delta_rule, hattention_kernel,
    hattention_prefill, hattention_step, num_levels_required)
from .geo import (  # noqa: F401
    get_geo_shift, get_regions, hept_positions, pad_to_multiple, quantile_partition, region_inputs, row_range)
from .bucket_attn import hept_attention_core, hept_bucket_attention, prep_qk, qkv_res  # noqa: F401
from .layer import (  # noqa: F401
    FusedRMSNormGated, ShortConvolution, add_rms_norm, compute_lambda, gate_inputs, rms_norm_gated)
from .lsh import (  # noqa: F401
    E2LSH, LSHOrdering, batched_index_select, invert_permutation, lsh_bucket_sort, lsh_hash, lsh_mapping,
    permute_rows, segmented_sort, sort_to_buckets, unsort_from_buckets)

__all__ = [
    "LampaError", "check_status", "HState", "HStruct", "HType", "hattention_prefill", "hattention_step", "chunk_gated_delta_rule", "chunk_h_gated_delta_rule",
    "hattention_kernel", "num_levels_required", "E2LSH", "LSHOrdering", "batched_index_select",
    "invert_permutation", "lsh_bucket_sort", "lsh_hash", "lsh_mapping", "permute_rows", "segmented_sort",
    "sort_to_buckets", "unsort_from_buckets", "qkv_res", "prep_qk", "hept_bucket_attention", "hept_attention_core",
    "get_geo_shift", "get_regions", "hept_positions", "pad_to_multiple",
    "quantile_partition", "region_inputs", "row_range", "FusedRMSNormGated", "ShortConvolution", "compute_lambda",
    "gate_inputs", "rms_norm_gated", "add_rms_norm",
]
