"""VSA2 on B200: the `echosparse.vsa` entry points (reference: echosparse/vsa/__init__.py:9-15) over the native kernels.

`vsa2_attention` takes the preblocked [B, H, NB*64, D] layout; `layout` maps real tokens to it and back. Importing this
package needs neither a GPU nor the native library; the first call loads it and fails loudly when it is missing.
"""
from .layout import BlockLayout, build_layout, from_blocked, sequence_layout, to_blocked
from .tiers import RepTiers, TierSelection, rep_fine_attention, route_tiers
from .ops import (Selection, SplitKV, SplitPolicy, describe_split, fine_block_sparse_attention, mask_to_selection,
                  resolve_bwd_variant, route, route_rows, set_bwd_variant, set_tk_bwd_opts, vsa2_attention, vsa_attention)

__all__ = ["BlockLayout", "Selection", "build_layout", "fine_block_sparse_attention", "from_blocked", "mask_to_selection",
           "route", "sequence_layout", "to_blocked", "vsa2_attention", "SplitKV", "SplitPolicy", "describe_split", "RepTiers", "TierSelection",
           "rep_fine_attention", "route_tiers", "route_rows", "vsa_attention", "resolve_bwd_variant", "set_bwd_variant",
           "set_tk_bwd_opts"]
