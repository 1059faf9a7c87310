"""prima.cpp_b200 — B200-native (sm_100a) quantized-decode hot path of prima.cpp behind a C ABI.

The product is ``libprima_b200.so`` (CUDA kernels + C++ decode engine, ``include/prima_b200.h``) and
``libggml-b200.so`` (the same kernels behind the reference's ggml-backend vtables, ``include/ggml_b200.h``).
The same library and model object serve a second family of models, the layer list: dense bf16 / f32 weights from a safetensors
directory, sequence slots and a ragged batch step (``Model.from_dir`` / ``Model.batch_step``), driven by :class:`BatchScheduler`.
Designs: Vamidra (windowed attention with kept first tokens, Mamba-2 mixers), Mumizen (decay linear attention, attention over a
low-rank latent, clamped gated feed-forward and mixtures of experts, token shift, depth average), Sapudra (post-norm layers with a
position table, windowed attention with normed query / key heads, squared-ReLU feed-forward, router with sigmoid scores and expert groups)
and Zevedra (dual mixers: windowed or sink attention beside the gated delta rule or HGRN2, bigram embedding, experts weighted on their input).
This Python package is only the thin ctypes binding plus the schedulers; it never falls back to a CPU path: importing
:mod:`host` raises if the CUDA library is missing.
"""
from .host import Lib, Model, HParams, lib_path, build, TYPES  # noqa: F401
from .scheduler import BatchScheduler, Request  # noqa: F401
from .pipeline import PipelineRunner, RingRunner, PrefillPipeline, layer_windows  # noqa: F401
