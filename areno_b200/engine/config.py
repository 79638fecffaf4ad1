"""Engine configuration: optimizer schedule, runtime allocation, model architecture, layout.

Field names follow the reference's dataclasses (``areno/engine/config.py:26-238``) so that
``ArenoConfig(optimizer={...}, runtime={...})`` dictionaries written for it keep working; the
runtime knobs that only made sense for its kernels (``attn_backend``) are accepted and ignored
where noted, and B200-specific knobs are added (``kv_dtype``, ``train_sharding``, ``rollout_tp``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Literal

import torch


_DTYPE_NAMES: dict[str, torch.dtype] = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
}


def parse_dtype(value: Any, default: torch.dtype = torch.bfloat16) -> torch.dtype:
    """Floating-point dtype named by a checkpoint's ``config.json`` (``torch_dtype`` / ``dtype``): the long names, the
    usual short forms and a ``torch.`` prefix are accepted, ``None`` or an empty string gives ``default``, and a name
    that is not a floating-point dtype this framework computes in is an error instead of a silent bf16
    (``areno/engine/config.py:286``)."""
    if value is None or value == "":
        return default
    if isinstance(value, torch.dtype):
        if value not in _DTYPE_NAMES.values():
            raise ValueError(f"unsupported model dtype {value}")
        return value
    key = str(value).strip().lower()
    if key.startswith("torch."):
        key = key[len("torch."):]
    if key not in _DTYPE_NAMES:
        raise ValueError(f"unsupported model dtype {value!r}; one of {sorted(_DTYPE_NAMES)}")
    return _DTYPE_NAMES[key]


@dataclass
class OptimizerConfig:
    lr: float = 1e-4
    min_lr: float = 0.0
    lr_decay_steps: int = 0
    lr_warmup_steps: int = 0
    lr_decay_style: Literal["constant", "linear", "cosine"] = "constant"
    betas: tuple[float, float] = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.0
    grad_clip_norm: float | None = None
    adam_8bit: bool = False
    # elements per flat gradient/optimizer bucket (reduce-scatter granularity)
    fp32_master_bucket_numel: int = 64 * 1024 * 1024


@dataclass
class RuntimeConfig:
    kv_block_size: int = 64               # accepted for compatibility (checked, not read): pages hold 64 tokens
    kv_dtype: Literal["bf16", "fp8"] = "bf16"
    attn_backend: str = "flash"           # accepted for compatibility; one kernel family exists here
    activation_checkpointing: bool = True
    keep_rollout_state: bool = True
    eager_decode: bool = False
    decode_graph_buckets: list[int] = field(
        default_factory=lambda: [1, 2, 4, 8, 12, 16, 24, 32, 40, 48, 56, 64, 96, 128, 192, 256, 384, 512]
    )
    max_prefill_tokens: int = 16384
    kv_cache_fraction: float = 0.9        # accepted for compatibility: the KV pool is running sequences x longest sequence
    max_model_len: int | None = None
    logprob_chunk: int = 4096             # rows per lm_head + log-prob chunk
    # training at tp_size > 1: shard the activations between the TP seams by tokens (all-gather + reduce-scatter in
    # place of the all-reduces); ARENO_SEQUENCE_PARALLEL=1 switches it on as well
    sequence_parallel: bool = False
    deterministic: bool = False           # accepted for compatibility: the kernels' reductions run in a fixed order anyway

    def __post_init__(self) -> None:
        if self.attn_backend not in {"flash", "native"}:
            raise ValueError("runtime.attn_backend must be one of: flash, native")
        if self.kv_dtype not in {"bf16", "fp8"}:
            raise ValueError("runtime.kv_dtype must be one of: bf16, fp8")


@dataclass
class ModelConfig:
    """Normalised architecture description derived from a HF ``config.json`` by a model adapter."""

    model_type: str = "qwen3"
    checkpoint_prefix: str = "model"
    checkpoint_lm_head_key: str = "lm_head.weight"
    vocab_size: int = 151936
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = False
    qkv_bias: bool = False
    qk_norm: bool = True
    v_norm: bool = False
    dtype: torch.dtype = torch.bfloat16
    hidden_act: str = "silu"
    layer_types: tuple[str, ...] | None = None
    sliding_window: int | None = None
    swa_head_dim: int | None = None
    swa_num_key_value_heads: int | None = None
    rope_parameters: dict[str, dict[str, Any]] | None = None
    attention_k_eq_v: bool = False
    num_kv_shared_layers: int = 0
    hidden_size_per_layer_input: int = 0
    vocab_size_per_layer_input: int | None = None
    use_double_wide_mlp: bool = False
    enable_moe_block: bool = False
    use_bias: bool = False
    layer_group_size: int = 1
    partial_rotary_factor: float = 1.0
    num_experts: int | None = None
    num_experts_per_tok: int = 1
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    first_k_dense_replace: int = 0
    moe_intermediate_size: int = 0
    num_shared_experts: int | None = None
    shared_expert_intermediate_size: int = 0
    moe_router_enable_expert_bias: bool = True
    norm_topk_prob: bool = True
    moe_router_dtype: torch.dtype = torch.float32
    score_function: str = "sigmoid"
    topk_method: str = "noaux_tc"
    group_norm_size: int = 128
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    kv_lora_rank: int | None = None
    linear_scale: bool = True
    linear_silu: bool = False
    sequence_parallel: bool = False
    moe_router_bias_update_rate: float = 0.0
    attention_softmax_scale: float | None = None
    final_logit_softcapping: float | None = None
    attn_output_gate: bool = False
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 16
    embed_scale: float = 1.0
    rope_interleaved: bool = False
    norm_weight_offset: float = 0.0   # Gemma-style (1 + w) norms use 1.0
    # Fields of the reference's ``ModelConfig`` that select among its back ends or describe layers this framework
    # does not execute (multi-token-prediction heads): accepted so that configs written for it construct, not read.
    num_nextn_predict_layers: int = 0
    mtp_loss_scaling_factor: float = 0.0
    linear_backend: str | None = None
    moe_backend: str | None = None
    attn_backend: str | None = None
    extra: dict[str, Any] = field(default_factory=dict)

    @property
    def rotary_dim(self) -> int:
        rot = int(self.head_dim * self.partial_rotary_factor)
        return rot - (rot % 2)

    def kv_replication(self, tp_size: int) -> int:
        """How many TP ranks share one KV head (1 when kv heads divide evenly)."""
        if tp_size <= self.num_key_value_heads:
            return 1
        return tp_size // self.num_key_value_heads

    def validate_tp(self, tp_size: int, inference_only: bool = False) -> None:
        """Shapes must split evenly over TP; KV heads may instead be replicated when ``tp_size`` is a
        multiple of them (the reference allows that only for three families,
        ``areno/engine/config.py:159-171``).  A layout that is used for inference only (a separate rollout
        layout) may also be wider than the query heads divide, as long as it is a multiple of the KV heads: the
        query heads of one KV group are then dealt out unevenly over the ranks that share the group's KV head
        and the short ranks carry zero-weight padding heads (28 query / 4 KV heads at tp 8: 4 + 3 per pair)."""
        if tp_size < 1:
            raise ValueError("tp_size must be >= 1")
        kv = self.num_key_value_heads
        if self.num_attention_heads % tp_size != 0:
            padded_ok = (inference_only and self.model_type in ("llama", "qwen2", "qwen3") and kv > 0
                         and tp_size % kv == 0 and self.num_attention_heads % kv == 0)
            if not padded_ok:
                raise ValueError(
                    f"num_attention_heads={self.num_attention_heads} must be divisible by tp_size={tp_size}")
        if kv % tp_size != 0 and tp_size % kv != 0:
            raise ValueError(f"num_key_value_heads={kv} must divide or be divisible by tp_size={tp_size}")
        if self.intermediate_size and self.intermediate_size % tp_size != 0:
            raise ValueError(f"intermediate_size={self.intermediate_size} must be divisible by tp_size={tp_size}")
        if self.num_experts and self.num_experts % tp_size != 0:
            raise ValueError(f"num_experts={self.num_experts} must be divisible by tp_size={tp_size}")


@dataclass
class EngineConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    runtime: RuntimeConfig = field(default_factory=RuntimeConfig)
    model_path: str = ""
    tp_size: int = 1
    dp_size: int | None = None
    # TP width of the rollout engine when it differs from training (None: same layout).  Requires the
    # training layout to be pure data parallel (tp_size == 1): every rank then owns a full replica and
    # cuts its rollout shard locally.
    rollout_tp_size: int | None = None
    # Expert parallelism for mixture-of-experts models: the experts are dealt out over the data-parallel ranks and
    # tokens are exchanged with their owners in every MoE layer, in training and in rollout alike (tp_size 1).
    expert_parallel: bool = False
    devices: list[int] | None = None
    dummy_load: bool = False
    max_running_seqs: int = 64
    decode_progress_interval_s: float = 10.0
    seed: int = 0
    backend: Literal["nccl", "gloo"] | None = None
    # ``loss_fn(data_pack, logprobs) -> loss | (loss, metrics)`` for packs that do not carry their own ``_loss_fn``
    # (the reference's way of handing the loss to the engine; ``ArenoEngine(config, loss_fn=...)`` is the other)
    train_loss_fn: Any = None

    def __post_init__(self) -> None:
        if isinstance(self.optimizer, dict):
            self.optimizer = OptimizerConfig(**self.optimizer)
        if isinstance(self.runtime, dict):
            self.runtime = RuntimeConfig(**self.runtime)
        if self.devices is None:
            n = self.tp_size * (self.dp_size or 1)
            self.devices = list(range(n))
        world = len(self.devices)
        if self.tp_size < 1 or world % self.tp_size != 0:
            raise ValueError(f"world size {world} must be a positive multiple of tp_size={self.tp_size}")
        if self.dp_size is None:
            self.dp_size = world // self.tp_size
        if self.dp_size * self.tp_size != world:
            raise ValueError(f"tp_size*dp_size = {self.tp_size * self.dp_size} does not match {world} devices")
        self.model.validate_tp(self.tp_size)
        if self.rollout_tp_size is not None and self.rollout_tp_size != self.tp_size:
            if self.tp_size != 1:
                raise ValueError("rollout_tp_size requires tp_size == 1 for training")
            if self.rollout_tp_size < 1 or world % self.rollout_tp_size != 0:
                raise ValueError(f"world size {world} must be a multiple of rollout_tp_size={self.rollout_tp_size}")
            self.model.validate_tp(self.rollout_tp_size, inference_only=True)
        if self.expert_parallel:
            if self.tp_size != 1 or self.rollout_tp_size not in (None, 1):
                raise ValueError("expert_parallel shards the experts over the data-parallel group: tp_size must be 1")
            if not self.model.num_experts or self.model.num_experts % world != 0:
                raise ValueError(f"expert_parallel needs num_experts divisible by the {world} ranks")
        if self.runtime.kv_block_size % 16 != 0:
            raise ValueError("runtime.kv_block_size must be a multiple of 16")

    @property
    def world_size(self) -> int:
        return len(self.devices or [])

    @property
    def rollout_tp(self) -> int:
        return int(self.rollout_tp_size or self.tp_size)

    @property
    def rollout_dp(self) -> int:
        return self.world_size // self.rollout_tp
