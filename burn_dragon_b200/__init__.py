"""burn_dragon_b200: a Blackwell-native (sm_100a) training and inference framework for the Dragon
Hatchling (BDH) language model family, with the capabilities of mosure/burn_dragon.

Layout:
  config      layered TOML configuration (same schema and merge rules as the reference)
  data        tokenizers, datasets, batch samplers
  models      BDH (recurrent / chunked / row-normalised parallel paths), Mamba-2, Mamba-3, BDH-graph
  ops         Python front ends of the hand-written CUDA kernels plus their fp32 torch definitions
  parallel    DDP / FSDP / neuron-sharded TP, symmetric memory, watchdog
  engine      trainer, generator, checkpoints (native + Burn record), metrics, bench harness
  csrc        CUDA / C++ sources of the extension
"""
__version__ = "0.1.0"
