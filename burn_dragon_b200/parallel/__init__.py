"""Data / parameter / neuron-sharded parallelism over NCCL and NVLink peer memory.

    ddp   engine.trainer.Trainer + parallel.ddp.DataParallel (flat gradient buffer, fused all-reduce)
    fsdp  parallel.fsdp.FSDP   (sharded master weights / moments / gradient reduction)
    tp    parallel.tp.NeuronTP (each rank owns a slice of every head's neurons)
"""


def build_wrapper(model, cfg, strategy: str):
    """FSDP / TP wrapper for `model` from a TrainingConfig."""
    o = cfg.optimizer
    kw = dict(lr=o.learning_rate, weight_decay=o.weight_decay, beta1=o.beta1, beta2=o.beta2, eps=o.eps,
              fused=cfg.parallel.fused_collectives)
    if strategy == "fsdp":
        from .fsdp import FSDP
        return FSDP(model, **kw)
    if strategy == "tp":
        from ..models.bdh import BDH
        from .tp import NeuronTP
        if type(model) is not BDH:
            raise ValueError(f"parallel.strategy = \"tp\" shards the neurons of a BDH model; {type(model).__name__} "
                             "trains under \"ddp\" or \"fsdp\"")
        return NeuronTP(model, **kw)
    raise ValueError(f"no wrapper for strategy {strategy}")
