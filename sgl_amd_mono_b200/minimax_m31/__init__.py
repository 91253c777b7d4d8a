"""FFN-only launch after SGLang's attention (reference: ``sgl_amd_mono/minimax_m31``):
RMSNorm, fp32 sigmoid router with top-k renormalised, MXFP4 routed experts on MXFP8
activations and one shared expert.  BASELINE config 1 is this block at hidden 2048, 64
experts top-4, intermediate 768 with plain SwiGLU and a bf16 shared expert."""

HF_CONFIG = dict(hidden_size=2048, n_routed_experts=64, num_experts_per_tok=4, moe_intermediate_size=768,
                 routed_scaling_factor=1.0, scoring_func="sigmoid", rms_norm_eps=1e-6)
