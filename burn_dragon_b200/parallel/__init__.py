"""Data / parameter / neuron-sharded parallelism over NCCL and NVLink peer memory."""
