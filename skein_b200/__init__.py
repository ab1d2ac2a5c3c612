"""skein_b200: a Blackwell-native LLM serving compiler and runtime (B200, sm_100a, NVLink 5).

Sub-packages
    ops       operator interface: hand-written CUDA kernels on GPU, PyTorch fp32 references on CPU
    models    Mixtral / Llama decoder graphs written against the operator interface
    runtime   paged KV, continuous batching engine, CUDA-graph manager, HTTP server, metrics
    parallel  tensor / expert / pipeline parallel plumbing over torch.distributed + peer memory
    planner   IR, cost model, placement search (C++ core with Python bindings)
    cli       the `skein` command: extract | compile | verify | serve | calibrate | bench
"""
__version__ = "0.1.0"
