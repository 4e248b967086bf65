"""Native single-YAML schema: ``parallel / data / model / features / training / tools``.

Same keys as the reference's native trainer (mindspeed_mm/fsdp/params/{parallel_args,training_args,
feature_args,model_args,data_args,lora_args,tools_args}.py; example examples/qwen3_5/qwen3_5_35B_config.yaml),
validated with pydantic.  Unknown keys are kept (``extra="allow"``) so that model- or dataset-specific
options flow through to the plugin that understands them.  ``load_config(path, overrides)`` applies
``a.b.c=value`` command-line overrides (mindspeed_mm/config/config_manager.py:575-603) on top of the YAML.
"""
from __future__ import annotations

import os
import re
from typing import Any, Dict, List, Literal, Optional, Sequence, Union

import yaml
from pydantic import BaseModel, ConfigDict, Field, model_validator


class _Base(BaseModel):
    model_config = ConfigDict(extra="allow", validate_assignment=True, protected_namespaces=())

    def get(self, key, default=None):
        return getattr(self, key, default)


# ------------------------------------------------------------------------------------------ parallel
class FSDPPlan(_Base):
    ignored_modules: List[str] = Field(default_factory=list)
    apply_modules: List[str] = Field(default_factory=list)
    hook_modules: Optional[List[str]] = None
    param_dtype: Optional[str] = "bf16"
    reduce_dtype: Optional[str] = "fp32"
    output_dtype: Optional[str] = None
    cast_forward_inputs: bool = True
    reshard_after_forward: bool = True
    num_to_forward_prefetch: Optional[int] = 1
    num_to_backward_prefetch: Optional[int] = 1
    pregather: bool = False
    cpu_offload: bool = False
    comm: Literal["auto", "p2p", "nccl"] = "auto"     # auto: NVLink peer kernels when symmetric memory is available


class TPPlan(_Base):
    colwise_parallel: List[str] = Field(default_factory=list)
    rowwise_parallel: List[str] = Field(default_factory=list)
    sequence_parallel: List[str] = Field(default_factory=list)


class EPPlan(_Base):
    apply_modules: List[str] = Field(default_factory=list)
    dispatcher: Literal["alltoall", "allgather", "mc2", "p2p", "fused"] = "alltoall"
    apply_efsdp_modules: List[str] = Field(default_factory=list)
    use_npu_fused_ops: bool = True          # accepted for recipe compatibility; ignored


class RecomputePlan(_Base):
    apply_modules: List[str] = Field(default_factory=list)
    use_reentrant: bool = False


class ParallelArguments(_Base):
    data_parallel_size: Optional[int] = None
    data_parallel_replicate_size: int = 1
    fully_shard_parallel_size: Union[str, int] = "auto"
    fsdp_plan: FSDPPlan = Field(default_factory=FSDPPlan)
    tensor_parallel_size: int = 1
    tp_plan: TPPlan = Field(default_factory=TPPlan)
    pipeline_parallel_size: int = 1
    ring_attention_size: int = 1
    ulysses_parallel_size: int = 1
    expert_parallel_size: int = 1
    expert_fully_shard_parallel_size: Optional[int] = None
    ep_plan: EPPlan = Field(default_factory=EPPlan)
    recompute: bool = False
    recompute_plan: RecomputePlan = Field(default_factory=RecomputePlan)

    def resolve(self, world_size: int) -> "ParallelArguments":
        """World-size dependent defaults and consistency checks (parallel_args.py:98-152).  Unlike the
        reference, tensor parallelism and ring attention are accepted here."""
        tp, pp = self.tensor_parallel_size, self.pipeline_parallel_size
        cp = self.ring_attention_size * self.ulysses_parallel_size
        if world_size % (tp * pp * cp):
            raise ValueError(f"World size should be a multiple of tensor_parallel_size: {tp}, pipeline_parallel_size: "
                             f"{pp}, ulysses_parallel_size: {self.ulysses_parallel_size}, ring_attention_size: "
                             f"{self.ring_attention_size}.")
        if self.fully_shard_parallel_size == "auto":
            self.fully_shard_parallel_size = world_size // (tp * pp * self.data_parallel_replicate_size)
        self.fully_shard_parallel_size = int(self.fully_shard_parallel_size)
        if world_size % (tp * pp * self.fully_shard_parallel_size):
            raise ValueError("World size should be a multiple of tensor_parallel_size x fully_shard_parallel_size.")
        if self.fully_shard_parallel_size < cp:
            raise ValueError("fully shard parallel size should be greater the ring_attention_size * ulysses_parallel_size.")
        dp = world_size // (tp * pp * cp)
        if self.data_parallel_size is None:
            self.data_parallel_size = dp
        if self.data_parallel_size != dp:
            raise ValueError(f"data_parallel_size should be {dp} for this world size and tp/pp/cp.")
        if self.expert_fully_shard_parallel_size is None:
            self.expert_fully_shard_parallel_size = world_size // pp // self.expert_parallel_size
        return self

    def state_kwargs(self) -> Dict[str, Any]:
        """Arguments for ``parallel.state.init_parallel_state``."""
        cp = self.ring_attention_size * self.ulysses_parallel_size
        return dict(pipeline_parallel_size=self.pipeline_parallel_size,
                    data_parallel_replicate_size=self.data_parallel_replicate_size,
                    fully_shard_parallel_size=int(self.fully_shard_parallel_size) // cp
                    if self.fully_shard_parallel_size != "auto" else "auto",
                    ring_attention_size=self.ring_attention_size, ulysses_parallel_size=self.ulysses_parallel_size,
                    tensor_parallel_size=self.tensor_parallel_size, expert_parallel_size=self.expert_parallel_size)


# ------------------------------------------------------------------------------------------ data
class DatasetArguments(_Base):
    dataset_type: str = "huggingface"
    basic_parameters: Dict[str, Any] = Field(default_factory=dict)
    preprocess_parameters: Optional[Dict[str, Any]] = Field(default_factory=dict)
    attr: Dict[str, Any] = Field(default_factory=dict)


class CollateArguments(_Base):
    collator_id: Optional[str] = None
    model_name: Optional[str] = None
    ignore_pad_token_for_loss: bool = True
    pad_to_multiple_of: int = 1


class DataloaderArguments(_Base):
    dataloader_mode: str = "sampler"
    sampler_type: str = "BaseRandomBatchSampler"
    shuffle: Optional[bool] = True
    drop_last: bool = True
    pin_memory: bool = True
    collate_param: CollateArguments = Field(default_factory=CollateArguments)
    num_workers: int = 2
    enable_preload: bool = False
    max_seq_len: Optional[int] = None             # dynamic (packed) batching budget
    dynamic_batch_buffer_size: int = 200


class DataArguments(_Base):
    dataset_param: DatasetArguments = Field(default_factory=DatasetArguments)
    val_dataset_param: Optional[DatasetArguments] = None
    dataloader_param: DataloaderArguments = Field(default_factory=DataloaderArguments)


# ------------------------------------------------------------------------------------------ model / lora
class ModelArguments(_Base):
    model_id: Optional[str] = None
    model_name_or_path: Optional[str] = None
    trust_remote_code: bool = False
    attn_implementation: Optional[str] = "flash_attention_2"
    freeze: List[str] = Field(default_factory=list)
    mtp_num_layers: int = 0
    mtp_loss_scaling_factor: float = 0.1


class LoraArguments(_Base):
    enable: bool = False
    rank: int = 8
    alpha: int = 16
    target_modules: List[str] = Field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj"])
    dropout: float = 0.0
    init_lora_weights: Union[bool, str] = True
    pretrained_lora_path: Optional[str] = None


# ------------------------------------------------------------------------------------------ features
class LossArguments(_Base):
    loss_type: Optional[str] = "default"
    router_aux_loss_coef: float = 0.0
    router_aux_loss_offload: bool = False


class ChunkLossPlan(_Base):
    apply_module: str = "lm_head"
    chunk_size: int = 1024
    total_chunk_size: Optional[int] = None


class ActivationOffloadPlan(_Base):
    apply_modules: List[str] = Field(default_factory=list)


class ChunkMbsPlan(_Base):
    apply_modules: List[str] = Field(default_factory=list)
    chunk_mbs: int = 1
    batch_dim: int = 0
    chunk_arg_indexs: List[int] = Field(default_factory=lambda: [0])
    chunk_kwarg_names: List[str] = Field(default_factory=list)


class EPBalancePlan(_Base):
    max_dup_experts_num: int = 2


class FeatureArguments(_Base):
    recompute: bool = False
    recompute_plan: RecomputePlan = Field(default_factory=RecomputePlan)
    loss_cfg: LossArguments = Field(default_factory=LossArguments)
    enable_chunk_loss: bool = False
    enable_dynamic_chunk_loss: bool = False
    chunkloss_plan: ChunkLossPlan = Field(default_factory=ChunkLossPlan)
    enable_activation_offload: bool = False
    activation_offload_plan: ActivationOffloadPlan = Field(default_factory=ActivationOffloadPlan)
    enable_chunk_mbs: bool = False
    chunkmbs_plan: ChunkMbsPlan = Field(default_factory=ChunkMbsPlan)
    enable_ep_balance: bool = False
    ep_balance_plan: EPBalancePlan = Field(default_factory=EPBalancePlan)
    skip_moe_pad_tokens: bool = False


# ------------------------------------------------------------------------------------------ training
class LRScalingPlan(_Base):
    match: str = ""
    scale: float = 1.0


class TrainingArguments(_Base):
    lora: LoraArguments = Field(default_factory=LoraArguments)
    lr: float = 1e-5
    lr_min: float = 1e-7
    lr_start: float = 0.0
    weight_decay: float = 0.0
    no_decay_modules: List[str] = Field(default_factory=list)
    no_decay_params: List[str] = Field(default_factory=lambda: ["bias"])
    optimizer: Literal["adamw", "adamw_swap", "muon"] = "adamw"
    mem_fraction_static: float = 0.9
    matched_adamw_rms: float = 0.2
    muon_momentum: float = 0.95
    ns_steps: int = 5
    adam_fused: bool = True
    use_ema: bool = False               # moving average of the master weights (saved with the checkpoint; exported last)
    ema_decay: float = 0.9999
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8
    clip_grad: float = 0.0
    clip_grad_ema_decay: float = 0.0    # > 0: adaptive clipping (threshold = moving average of the norm + 3 sigma)
    clip_grad_foreach: bool = True
    micro_batch_size: int = 1
    gradient_accumulation_steps: Optional[int] = 1
    global_batch_size: Optional[int] = None
    lr_warmup_ratio: float = 0.0
    lr_decay_style: str = "cosine"
    lr_decay_ratio: float = 1.0
    enable_full_determinism: bool = False
    save_async: bool = False
    save_ckpt_dtype: Optional[Literal["fp32", "fp16", "bf16"]] = None
    seed: int = 42
    init_model_with_meta_device: bool = True
    train_iters: int = 10
    train_epochs: Optional[int] = None
    load: Optional[str] = None
    load_format: Literal["auto", "hf", "dcp", "sharded"] = "auto"
    save_format: Literal["auto", "hf", "dcp", "sharded"] = "dcp"
    load_strict: bool = True
    no_load_optim: bool = False
    no_load_rng: bool = False
    save: Optional[str] = None
    no_save_optim: bool = False
    no_save_rng: bool = False
    log_interval: int = 1
    save_interval: int = 0
    val_interval: int = 0
    val_micro_batch_size: Optional[int] = None
    manual_gc_interval: int = 0
    use_deter_comp: bool = False
    plugin: List[str] = Field(default_factory=list)
    lr_scaling_plan: Optional[List[LRScalingPlan]] = None
    exit_interval: int = 0
    exit_duration_in_mins: float = 0.0
    watchdog_timeout_s: float = 0.0


# ------------------------------------------------------------------------------------------ tools
class StaticParam(_Base):
    level: str = "level1"
    with_stack: bool = False
    with_memory: bool = False
    record_shapes: bool = False
    with_cpu: bool = True
    save_path: str = "./profiling"
    start_step: int = 10
    end_step: int = 11
    data_simplification: bool = False
    aic_metrics_type: str = "PipeUtilization"     # accepted for recipe compatibility; no meaning on a GPU
    analyse_flag: bool = False


class ProfilerArguments(_Base):
    enable: bool = False
    profile_type: str = "static"
    ranks: List[int] = Field(default_factory=lambda: [0])
    static_param: StaticParam = Field(default_factory=StaticParam)


class MemoryProfilerArguments(_Base):
    enable: bool = False
    start_step: int = 1
    end_step: int = 2
    save_path: str = "./memory_snapshot"
    dump_ranks: List[int] = Field(default_factory=lambda: [0])
    stacks: Literal["python", "all"] = "all"
    max_entries: Optional[int] = None
    mem_info: bool = False


class ToolsArguments(_Base):
    profile: ProfilerArguments = Field(default_factory=ProfilerArguments)
    memory_profile: MemoryProfilerArguments = Field(default_factory=MemoryProfilerArguments)
    tensorboard_dir: Optional[str] = None          # scalars per iteration (loss, lr, grad norm, router aux loss, memory)
    tensorboard_log_interval: int = 1
    wandb_project: Optional[str] = None
    wandb_exp_name: Optional[str] = None
    wandb_save_dir: Optional[str] = None


class Arguments(_Base):
    parallel: ParallelArguments = Field(default_factory=ParallelArguments)
    data: DataArguments = Field(default_factory=DataArguments)
    model: ModelArguments = Field(default_factory=ModelArguments)
    features: FeatureArguments = Field(default_factory=FeatureArguments)
    training: TrainingArguments = Field(default_factory=TrainingArguments)
    tools: ToolsArguments = Field(default_factory=ToolsArguments)

    @model_validator(mode="after")
    def _mirror_recompute(self):
        # older recipes put ``recompute`` under ``parallel`` and newer ones under ``features``
        if self.parallel.recompute and not self.features.recompute:
            self.features.recompute = True
            if not self.features.recompute_plan.apply_modules:
                self.features.recompute_plan = self.parallel.recompute_plan
        return self


# ------------------------------------------------------------------------------------------ loading
def _parse_value(s: str) -> Any:
    try:
        return yaml.safe_load(s)
    except yaml.YAMLError:
        return s


def apply_overrides(tree: Dict[str, Any], overrides: Sequence[str]) -> Dict[str, Any]:
    """``a.b.c=value`` items (list indices allowed: ``plugin.0=x``) are written into the dict tree."""
    for item in overrides:
        if item.endswith((".yaml", ".yml")) or "=" not in item or item.startswith("-"):
            continue
        key, val = item.split("=", 1)
        node = tree
        parts = key.strip().split(".")
        for p in parts[:-1]:
            if isinstance(node, list):
                node = node[int(p)]
            else:
                node = node.setdefault(p, {})
        last = parts[-1]
        if isinstance(node, list):
            node[int(last)] = _parse_value(val.strip())
        else:
            node[last] = _parse_value(val.strip())
    return tree


def load_config(path: Optional[str] = None, overrides: Sequence[str] = (), extra: Optional[Dict[str, Any]] = None,
                world_size: Optional[int] = None) -> Arguments:
    """YAML file -> validated ``Arguments``.  Priority: overrides > ``extra`` > YAML > defaults."""
    tree: Dict[str, Any] = {}
    if path:
        with open(path) as f:
            tree = yaml.safe_load(f) or {}
    if extra:
        _deep_update(tree, extra)
    apply_overrides(tree, overrides)
    args = Arguments(**tree)
    if world_size is None:
        world_size = int(os.environ.get("WORLD_SIZE", "1"))
    args.parallel.resolve(world_size)
    t = args.training
    if t.global_batch_size is None:
        t.global_batch_size = t.micro_batch_size * (t.gradient_accumulation_steps or 1) * args.parallel.data_parallel_size
    return args


def _deep_update(dst: Dict[str, Any], src: Dict[str, Any]) -> None:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _deep_update(dst[k], v)
        else:
            dst[k] = v


_WILD = re.compile(r"\{(\*|\d+(?:-\d+)?(?:,\d+(?:-\d+)?)*)\}")


def module_name_match(pattern: str, name: str) -> bool:
    """``model.layers.{*}.mlp`` style patterns: ``{*}`` is any index, ``{0-3,7}`` a set of indices
    (same pattern language as the reference's plans: models/transformers/base_model.py:63-141)."""
    rx, pos = "", 0
    sets = []
    for m in _WILD.finditer(pattern):
        rx += re.escape(pattern[pos:m.start()]) + r"(\d+)"
        sets.append(m.group(1))
        pos = m.end()
    rx += re.escape(pattern[pos:])
    mm = re.fullmatch(rx, name)
    if not mm:
        return False
    for spec, got in zip(sets, mm.groups()):
        if spec == "*":
            continue
        ok = False
        for part in spec.split(","):
            lo, _, hi = part.partition("-")
            if int(lo) <= int(got) <= int(hi or lo):
                ok = True
        if not ok:
            return False
    return True


def match_modules(patterns: Sequence[str], names: Sequence[str]) -> List[str]:
    return [n for n in names if any(module_name_match(p, n) for p in patterns)]
