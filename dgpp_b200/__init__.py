"""dgpp_b200: a Blackwell-datacenter (B200, sm_100a) native LLM inference engine.

Layers (top to bottom): ``serve`` (OpenAI-compatible HTTP) -> ``engine`` (scheduler glue, CUDA-graph
decode loop, paged KV) -> ``models`` (PyTorch definitions + reference paths) -> ``ops`` (hand-written
sm_100a kernels behind a C ABI) / ``parallel`` (tensor/expert parallel collectives over NVLink peer
memory) -> ``runtime`` (native C++ host runtime: scheduler, prefix cache, tokenizer, templates, ...).
"""
__version__ = "0.1.0"
