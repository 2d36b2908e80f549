"""onnx_genai_b200 -- a Blackwell-native generative-inference framework.

Same public surface as justinchuby/onnx-genai (ONNX model package + inference metadata, engine
with Sampler / SpeculativeProposer / DecodeBackend seams, OpenAI-compatible server, CLI, C API),
executed by hand-written sm_100a CUDA kernels driven from PyTorch.
"""
__version__ = "0.1.0"
