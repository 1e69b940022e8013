"""Layered TOML configuration.

Same schema and merge rules as the reference (src/config/train.rs:13-212, src/config/core.rs:6-53):
the first file is the base, every later file is deep-merged over it, and a table whose `type`
tag changes replaces the base table instead of merging into it. On top of the reference's
sections (`dataset`, `training`, `optimizer`, `generation`, `model`) this framework reads
`[parallel]`, `[precision]` and a few extra `[model]` keys (`kind`, `n_latent_per_head`,
`vocab_size`, and the Mamba / graph hyper-parameters).
"""
from __future__ import annotations

import copy
import dataclasses
import tomllib
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

ROTARY_KINDS = ("alibi", "rope", "pope")
MODEL_KINDS = ("bdh", "mamba2", "mamba3", "bdh_graph")
DATASET_TYPES = ("shakespeare", "hugging_face", "deep_math", "tiny_chat", "webscale_rl", "poetry_foundation",
                 "synthetic")
HF_FORMATS = ("jsonl", "text", "parquet", "csv")
LR_SCHEDULES = ("constant", "cosine", "linear", "exponential", "step", "noam")


class ConfigError(ValueError):
    pass


# ------------------------------------------------------------------------------------------------
# merge
# ------------------------------------------------------------------------------------------------
def merge_values(base: Any, overlay: Any) -> Any:
    """Deep-merge `overlay` into `base` and return the result (reference: config/train.rs:186-212).

    Tables merge key by key. If the overlay table carries a string `type` that differs from the
    base table's `type` (or the base has other keys but no `type`), the base table is emptied
    first. Anything that is not a pair of tables is replaced by the overlay value.
    """
    if isinstance(base, dict) and isinstance(overlay, dict):
        ov_type = overlay.get("type")
        if isinstance(ov_type, str):
            if "type" in base:
                changed = not (isinstance(base["type"], str) and base["type"] == ov_type)
            else:
                changed = len(base) > 0
            if changed:
                base.clear()
        for key, val in overlay.items():
            if key in base:
                base[key] = merge_values(base[key], val)
            else:
                base[key] = copy.deepcopy(val)
        return base
    return copy.deepcopy(overlay)


def load_value(path) -> Dict[str, Any]:
    p = Path(path)
    try:
        text = p.read_text()
    except OSError as e:
        raise ConfigError(f"failed to read configuration file {p}") from e
    try:
        return tomllib.loads(text)
    except tomllib.TOMLDecodeError as e:
        raise ConfigError(f"failed to parse {p} as TOML: {e}") from e


# ------------------------------------------------------------------------------------------------
# schema
# ------------------------------------------------------------------------------------------------
@dataclass
class TokenizerConfig:
    """reference: src/tokenizer/mod.rs:34-89. type = char{include_unknown} | byte{add_special_tokens}."""
    type: str = "char"
    include_unknown: bool = True
    add_special_tokens: bool = True
    vocab_path: Optional[str] = None


@dataclass
class DatasetConfig:
    cache_dir: str = "data"
    train_split_ratio: float = 0.9
    type: str = "shakespeare"
    url: Optional[str] = None
    # hugging_face
    repo_id: Optional[str] = None
    revision: Optional[str] = None
    format: str = "jsonl"
    train_files: List[str] = field(default_factory=lambda: ["train.jsonl"])
    validation_files: List[str] = field(default_factory=list)
    text_fields: List[str] = field(default_factory=lambda: ["text"])
    field_separator: str = "\n"
    template: Optional[str] = None
    max_records: Optional[int] = None
    # synthetic (uniform random bytes; what the benchmarks use)
    synthetic_tokens: int = 1 << 22
    seed: int = 0
    # keep the token array on the training device and gather the batches there (no per-step H2D copy)
    device_resident: bool = False
    tokenizer: TokenizerConfig = field(default_factory=TokenizerConfig)


@dataclass
class ContextStrategyConfig:
    type: str = "infinite"
    window: Optional[int] = None


@dataclass
class TrainingHyperparameters:
    block_size: int = 512
    batch_size: int = 24
    epochs: Optional[int] = None
    max_iters: int = 3000
    log_frequency: int = 100
    fast_train: bool = False
    context_strategy: ContextStrategyConfig = field(default_factory=ContextStrategyConfig)
    # additions
    seed: int = 1337
    grad_clip: Optional[float] = None
    grad_accum_steps: int = 1                # micro-batches of batch_size sequences per optimizer step
    checkpoint_every: Optional[int] = None   # steps; None = once per epoch like the reference
    recompute: Any = False                   # layers that re-run their forward in backward instead of saving
                                             # activations: false / true (none / all), a count, or "auto"
    attention_chunk: Optional[int] = None    # tokens per attention segment on the kernel path (states handed on
                                             # between segments); None = whole sequence; 1024 from 4096 tokens on when T > 1024 + 4 n_embd


@dataclass
class LearningRateScheduleConfig:
    type: str = "constant"
    initial_lr: Optional[float] = None
    min_lr: Optional[float] = None
    num_iters: Optional[int] = None
    final_lr: Optional[float] = None
    gamma: Optional[float] = None
    step_size: Optional[int] = None
    warmup_steps: Optional[int] = None
    model_size: Optional[int] = None


@dataclass
class OptimizerConfig:
    learning_rate: float = 1e-3
    weight_decay: float = 0.1
    lr_schedule: Optional[LearningRateScheduleConfig] = None
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-5


@dataclass
class GenerationConfig:
    prompt: str = ""
    max_tokens: Optional[int] = None
    temperature: float = 1.0
    top_k: Optional[int] = None
    context_strategy: ContextStrategyConfig = field(default_factory=ContextStrategyConfig)
    greedy: bool = False
    seed: int = 0


@dataclass
class ModelOverrides:
    """reference keys: src/config/core.rs:43-53; the rest are additions of this framework."""
    n_layer: Optional[int] = None
    n_embd: Optional[int] = None
    n_head: Optional[int] = None
    mlp_internal_dim_multiplier: Optional[int] = None
    relu_threshold: Optional[float] = None
    dropout: Optional[float] = None
    fused_kernels: Optional[bool] = None
    block_size: Optional[int] = None
    rotary_embedding: Optional[str] = None
    # additions
    kind: str = "bdh"
    n_latent_per_head: Optional[int] = None
    vocab_size: Optional[int] = None
    rope_theta: Optional[float] = None
    # mamba
    d_state: Optional[int] = None
    headdim: Optional[int] = None
    expand: Optional[int] = None
    chunk_size: Optional[int] = None
    d_conv: Optional[int] = None
    mimo_rank: Optional[int] = None
    # graph
    graph_block: Optional[int] = None
    graph_density: Optional[float] = None
    latent_active_blocks: Optional[List[int]] = None


@dataclass
class ParallelConfig:
    strategy: str = "single"        # single | ddp | fsdp | tp
    tp: int = 1                     # documentation of the intended group size; a tp job shards over all its ranks
    fused_collectives: bool = True  # in-kernel NVLink paths; False = NCCL-only baseline
    heartbeat_timeout_s: float = 60.0   # a peer silent for this long is reported before the next step; 0 = off


@dataclass
class PrecisionConfig:
    compute: str = "bf16"   # bf16 | fp32
    state: str = "fp32"     # decode state dtype


@dataclass
class TrainingConfig:
    dataset: DatasetConfig = field(default_factory=DatasetConfig)
    training: TrainingHyperparameters = field(default_factory=TrainingHyperparameters)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    generation: GenerationConfig = field(default_factory=GenerationConfig)
    model: ModelOverrides = field(default_factory=ModelOverrides)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    precision: PrecisionConfig = field(default_factory=PrecisionConfig)

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


_REQUIRED = {
    "dataset": ("cache_dir",),
    "training": ("block_size", "batch_size", "max_iters", "log_frequency"),
    "optimizer": ("learning_rate", "weight_decay"),
    "generation": ("prompt",),
}


def _build(cls, table: Dict[str, Any], where: str):
    if not isinstance(table, dict):
        raise ConfigError(f"[{where}] must be a table")
    names = {f.name: f for f in dataclasses.fields(cls)}
    kwargs = {}
    for key, val in table.items():
        if key not in names:
            raise ConfigError(f"unknown key `{key}` in [{where}]")
        kwargs[key] = val
    return cls(**kwargs)


def _context(table, where) -> ContextStrategyConfig:
    if table is None:
        return ContextStrategyConfig()
    cs = _build(ContextStrategyConfig, table, where)
    if cs.type not in ("infinite", "sliding"):
        raise ConfigError(f"[{where}] type must be `infinite` or `sliding`")
    if cs.type == "sliding" and not cs.window:
        raise ConfigError(f"[{where}] sliding context needs `window`")
    return cs


def from_dict(value: Dict[str, Any]) -> TrainingConfig:
    value = copy.deepcopy(value)
    for section, keys in _REQUIRED.items():
        if section not in value:
            raise ConfigError(f"missing section [{section}]")
        for k in keys:
            if k not in value[section]:
                raise ConfigError(f"missing field `{k}` in [{section}]")
    unknown = set(value) - {f.name for f in dataclasses.fields(TrainingConfig)}
    if unknown:
        raise ConfigError(f"unknown section(s): {sorted(unknown)}")

    ds = value["dataset"]
    tok = _build(TokenizerConfig, ds.pop("tokenizer", {}), "dataset.tokenizer")
    if tok.type not in ("char", "byte"):
        raise ConfigError("dataset.tokenizer.type must be `char` or `byte`")
    ds.setdefault("type", "shakespeare")
    dataset = _build(DatasetConfig, ds, "dataset")
    dataset.tokenizer = tok
    if dataset.type not in DATASET_TYPES:
        raise ConfigError(f"unknown dataset type `{dataset.type}`")
    if dataset.type == "hugging_face" and not dataset.repo_id:
        raise ConfigError("dataset type `hugging_face` needs `repo_id`")
    if dataset.format not in HF_FORMATS:
        raise ConfigError(f"unknown dataset format `{dataset.format}`")

    tr = value["training"]
    tr_ctx = _context(tr.pop("context_strategy", None), "training.context_strategy")
    training = _build(TrainingHyperparameters, tr, "training")
    training.context_strategy = tr_ctx
    if training.epochs is not None and training.epochs <= 0:
        training.epochs = None      # `epochs = 0` in an overlay switches back to max_iters

    op = value["optimizer"]
    sched = op.pop("lr_schedule", None)
    optimizer = _build(OptimizerConfig, op, "optimizer")
    if sched is not None:
        s = _build(LearningRateScheduleConfig, sched, "optimizer.lr_schedule")
        if s.type not in LR_SCHEDULES:
            raise ConfigError(f"unknown lr schedule `{s.type}`")
        if s.type == "linear" and s.final_lr is None:
            raise ConfigError("linear lr schedule needs `final_lr`")
        if s.type == "exponential" and s.gamma is None:
            raise ConfigError("exponential lr schedule needs `gamma`")
        if s.type == "step" and s.gamma is None:
            s.gamma = 0.1
        optimizer.lr_schedule = s

    ge = value["generation"]
    ge_ctx = _context(ge.pop("context_strategy", None), "generation.context_strategy")
    generation = _build(GenerationConfig, ge, "generation")
    generation.context_strategy = ge_ctx

    model = _build(ModelOverrides, value.get("model", {}), "model")
    if model.rotary_embedding is not None and model.rotary_embedding not in ROTARY_KINDS:
        raise ConfigError(f"rotary_embedding must be one of {ROTARY_KINDS}")
    if model.kind not in MODEL_KINDS:
        raise ConfigError(f"model.kind must be one of {MODEL_KINDS}")
    parallel = _build(ParallelConfig, value.get("parallel", {}), "parallel")
    if parallel.strategy not in ("single", "ddp", "fsdp", "tp"):
        raise ConfigError("parallel.strategy must be single | ddp | fsdp | tp")
    precision = _build(PrecisionConfig, value.get("precision", {}), "precision")
    if precision.compute not in ("bf16", "fp32"):
        raise ConfigError("precision.compute must be bf16 (kernels) or fp32 (torch path)")
    if precision.state != "fp32":
        raise ConfigError("precision.state: the recurrent decode state is kept in fp32 (no other type is implemented)")
    return TrainingConfig(dataset, training, optimizer, generation, model, parallel, precision)


def load_training_config(paths: Sequence) -> TrainingConfig:
    """Load and merge configuration files in order (reference: config/train.rs:157-176)."""
    if not paths:
        raise ConfigError("at least one configuration path is required")
    value = load_value(paths[0])
    for p in paths[1:]:
        value = merge_values(value, load_value(p))
    return from_dict(value)


PRESET_DIR = Path(__file__).resolve().parent.parent / "config"


def preset_path(name: str) -> Path:
    p = PRESET_DIR / f"{name}.toml"
    if not p.exists():
        raise ConfigError(f"no preset named `{name}` in {PRESET_DIR}")
    return p


def load_preset(*names: str) -> TrainingConfig:
    """`base.toml` first, then each named preset over it (how the reference's CLIs load configs)."""
    paths = [preset_path("base")] + [preset_path(n) for n in names if n != "base"]
    return load_training_config(paths)
