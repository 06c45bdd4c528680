"""Training primitives used by the quantisation-tuning tools (gradients of scales through frozen trellis cores)."""
