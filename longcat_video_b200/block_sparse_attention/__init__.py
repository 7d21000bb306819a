from .bsa_interface import flash_attn_bsa_3d  # noqa: F401
