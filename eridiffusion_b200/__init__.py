"""eridiffusion_b200 — a Blackwell (sm_100a) native diffusion-model training framework.

Layout: ``ops`` (CUDA kernels + PyTorch oracle), ``models``, ``adapters``, ``objectives``,
``optim``, ``parallel`` (NCCL + in-kernel NVLink paths), ``train``, ``data``, ``io``, ``config``,
``sampling``, ``memory``, ``serve``, ``cli``, ``utils``; native sources live in ``csrc``.
"""
__version__ = "0.1.0"
