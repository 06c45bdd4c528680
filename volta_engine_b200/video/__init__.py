"""Video diffusion transformer (MiniMax-H3 shape): INT8 rotated linears, the DiT block stack, sequence- and
tensor-parallel groups, the flow-matching denoise loop. See :mod:`.dit`."""
