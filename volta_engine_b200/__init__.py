"""volta_engine_b200: a Blackwell-native (sm_100a) LLM inference engine.

PyTorch is the framework layer (model definitions, loaders, paged-KV scheduler, CUDA-graph capture);
every hot op is a hand-written CUDA kernel in ``csrc/cuda`` built in-tree into
``_native/libvolta_kernels.so``; host-side runtime pieces (tokenizer, templates, HTTP front end, block
codecs) are C++ in ``csrc/host`` -> ``_native/libvolta_host.so``.
"""
__version__ = "0.1.0"
