"""Placeholder package of the reference's ``sgl_amd_mono/deepseek_v4`` model family.  Its
layer needs stages that are outside this build's hot-path scope (KV compressors, mHC
seams, KDA linear attention); the spec registers so that a server gets a clear refusal
instead of a silent fallback."""
