"""Host mirrors of the reference's `longcat_video/modules` pieces that touch the BSA path."""
from .attention import self_attention, self_attention_with_kv_cache  # noqa: F401
from .rope_3d import norm_rope, qk_norm_rope, qk_norm_rope_with_kv_cache, rms_norm, rope_table  # noqa: F401
