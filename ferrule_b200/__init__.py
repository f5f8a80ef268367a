"""ferrule_b200: a B200-native (sm_100a) exact LLM inference runtime.

Layers (bottom up): `csrc` hand-written CUDA kernels and C++ host runtime, `ops`
their launchers plus the PyTorch reference math, `models` the DeepSeek-family model
definitions, `parallel` tensor/expert/pipeline parallel plumbing over NCCL and
NVLink peer memory, `runtime` the scheduler / transaction / paged-KV / materialization
engine, `server` the OpenAI-compatible HTTP front end, `cli` the command line.
"""
__version__ = "0.2.0"
