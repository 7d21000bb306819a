from .bsa_interface import flash_attn_bsa_3d, flash_attn_bsa_3d_cond, flash_attn_bsa_3d_host  # noqa: F401
