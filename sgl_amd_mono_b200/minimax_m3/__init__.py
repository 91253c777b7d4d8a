"""GQA block-sparse attention + MXFP4 MoE layer (reference: ``sgl_amd_mono/minimax_m3``;
BASELINE config 4).  The block-sparse attention stage is not built yet; the spec refuses
with that reason while the MoE half is served by ``minimax_m31``'s launch."""
