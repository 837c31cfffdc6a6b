"""The reference's backend entry points (wall_x/fusions/backend.py) on this framework's kernels."""
from wallx_b200.ops.backend import (asym_dual_gmm_separated, get_rope_index, get_window_index, permute, rope, rope_bwd,  # noqa: F401
                                    rot_pos_emb, unpermute, unpermute_bwd)
