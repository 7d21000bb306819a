"""Host mirrors of the reference's `longcat_video/modules` pieces that touch the BSA path."""
from .rope_3d import qk_norm_rope, norm_rope, rope_table  # noqa: F401
