"""One spec per HF architecture: dispatches to the M3 or the M3.1 spec by the
checkpoint's quantisation (reference: ``sgl_amd_mono/minimax/spec.py:59-99``)."""
