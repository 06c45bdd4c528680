"""Weight / activation number formats: NVFP4, FP8 scalars, GGUF blocks, EXL3 trellis."""
