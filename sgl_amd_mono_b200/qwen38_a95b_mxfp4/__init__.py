"""Placeholder: the reference's ``sgl_amd_mono/qwen38_a95b_mxfp4`` registers nothing either."""
