"""prometheus_b200 — a Blackwell-native (B200, sm_100a) training framework.

Layers (bottom to top): ``ops`` (hand-written CUDA kernels bound with ctypes),
``kernels`` (numeric primitives API), ``model`` / ``latent`` (parameter tree and
forward), ``parallel`` (mesh, FSDP, EP, CP, PP over NCCL and peer memory),
``train`` (optimizer step on the tree), ``engine`` (the fused multi-GPU trainer),
``native`` (C++ checkpoint store, data loader, controller, observability, harness).
"""
__version__ = "0.1.0"
