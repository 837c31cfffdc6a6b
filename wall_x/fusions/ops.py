"""The reference's fused-op names (wall_x/fusions/ops.py) on this framework's kernels."""
from wallx_b200.ops.compat import (AsymmetricDualExpertGemm, MultimodalRoPE, PermuteMoE_topK, UnpermuteMoE_topK,  # noqa: F401
                                   asym_dual_gmm, get_rope_index, get_window_index, multimodal_rope, permute, rot_pos_emb,
                                   unpermute)
