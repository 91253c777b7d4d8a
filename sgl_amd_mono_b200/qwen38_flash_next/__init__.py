"""Placeholder: the reference's ``sgl_amd_mono/qwen38_flash_next`` registers nothing either."""
