"""Placeholder package of the reference's ``sgl_amd_mono/glm53_flash`` model family.  Its
layer needs stages that are outside this build's hot-path scope (KV compressors, mHC
seams, KDA linear attention); the spec registers so that a server gets a clear refusal
instead of a silent fallback."""
