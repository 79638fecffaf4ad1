"""Rank worker: one per GPU.  Owns the model shard, the inference engine, the training manager and
the auxiliary roles (reference / critic / reward models), and time-multiplexes the GPU between
them.  ``handle(op, payload)`` is the single entry point used by every cluster flavour (spawned
processes, in-process, SPMD under torchrun).

Counterpart of ``areno/engine/worker.py:54-467`` in the reference.  Differences that matter: the
decode loop has no per-step host sync (see ``inference.py``), gradients / optimizer state are
DP-sharded (see ``optim.py``), and the rollout engine reads the very buffers the optimizer writes,
so "weight sync" after a step is free when rollout and training share a layout.
"""

from __future__ import annotations

import json
import os
import time

import torch

from ..models import registry as model_registry
from ..parallel.context import get_context, use_context
from ..utils.log import get_logger
from ..utils.tracing import trace_range
from .config import EngineConfig
from .inference import InferenceEngine, RolloutOutput, SamplingParams
from .training import TrainingManager

logger = get_logger()


class RankWorker:
    def __init__(self, config: EngineConfig, device: torch.device | str | None = None):
        self.config = config
        from .. import configure_allocator

        configure_allocator()
        ctx = get_context()
        self.ctx = ctx
        self.device = torch.device(device) if device is not None else ctx.device
        t0 = time.time()
        self.adapter = model_registry.get_adapter(config.model.model_type)
        self.model = self.adapter.build(config.model, device=self.device)
        if config.dummy_load or not config.model_path:
            self.adapter.init_random(self.model, seed=config.seed)
        else:
            self.adapter.load_weights(self.model, config.model_path, config.model)
        # Rollout may use its own layout (e.g. tensor parallel while training is data parallel); it then
        # gets its own model instance whose shards are cut from the training replica after every step.
        self.rollout_ctx = ctx.rollout_layout
        if self.rollout_ctx is not ctx:
            if ctx.tp_size != 1:
                raise ValueError("a separate rollout layout requires the training layout to have tp_size == 1")
            with use_context(self.rollout_ctx):
                self.rollout_model = self.adapter.build(config.model, device=self.device)
            for p in self.rollout_model.parameters():
                p.requires_grad_(False)
        else:
            self.rollout_model = self.model
        self._rollout_stale = True
        self.tp_comm = None
        rctx = self.rollout_ctx
        if rctx.tp_size > 1 and self.device.type == "cuda" and os.environ.get("ARENO_TP_COMM", "fused") != "nccl":
            # peer-memory communicator for the fused GEMM -> all-reduce -> residual -> RMSNorm path
            from ..parallel.symm import setup_tp_comm

            # sized for the largest batch one forward pass can see: a prefill chunk or every decode slot of the group
            rows = max(int(config.runtime.max_prefill_tokens), int(config.max_running_seqs) * rctx.tp_size, 512)
            rows = min(rows, int(os.environ.get("ARENO_TP_COMM_MAX_ROWS", "16384")))
            self.tp_comm = setup_tp_comm(rctx, config.model.hidden_size, rows)
        self.trainer: TrainingManager | None = None
        self.infer: InferenceEngine | None = None
        self.roles = None
        self._resume_state_from = config.model_path if (config.model_path and not config.dummy_load) else None
        self._actor_on_device = True
        self.loss_fn = None
        logger.info("worker ready rank=%d tp=%d/%d dp=%d/%d build_s=%.2f", ctx.rank, ctx.tp_rank, ctx.tp_size,
                    ctx.dp_rank, ctx.dp_size, time.time() - t0)

    # ------------------------------------------------------------- components
    def training_manager(self) -> TrainingManager:
        if self.trainer is None:
            self.trainer = TrainingManager(self.model, self.config, self.device, loss_fn=self.loss_fn)
            if self.infer is not None:
                self.infer._graphs.clear()  # parameters were re-pointed into flat buckets
            src, self._resume_state_from = self._resume_state_from, None
            if src and os.path.isdir(os.path.join(src, "areno_state")):
                if self.load_training_state(src):
                    logger.info("resumed optimizer state and step counters from %s", src)
        return self.trainer

    def inference_engine(self, max_slots: int | None = None, max_model_len: int | None = None) -> InferenceEngine:
        rt = self.config.runtime
        slots = max_slots or self.config.max_running_seqs
        mlen = max_model_len or rt.max_model_len or min(self.config.model.max_position_embeddings, 8192)
        if self.infer is None or self.infer.max_slots < slots or self.infer.max_model_len < mlen:
            if self.infer is not None:
                self.infer.drop_kv_cache()
            self.infer = InferenceEngine(
                self.rollout_model, self.config.model.vocab_size, self.device, max_slots=slots, max_model_len=mlen,
                max_prefill_tokens=rt.max_prefill_tokens, kv_fp8=rt.kv_dtype == "fp8",
                graph_buckets=rt.decode_graph_buckets, eager=rt.eager_decode, seed=self.config.seed,
                max_new_cap=mlen, stream_salt=int(self.rollout_ctx.dp_rank))
        return self.infer

    # ---------------------------------------------------------------- rollout
    def sync_rollout_weights(self) -> int:
        """Bring the rollout model up to date with the trained parameters.  With a shared layout the
        engine reads the optimizer's own buffers and there is nothing to do; with a separate rollout
        layout every rank cuts its shard out of its local replica (no communication)."""
        if self.rollout_model is self.model or not self._rollout_stale:
            self._rollout_stale = False
            return 0
        from ..parallel.reshard import reshard_into

        with trace_range("weight_sync/reshard"):
            n = reshard_into(self.rollout_model, self.model, self.rollout_ctx.tp_rank, self.rollout_ctx.tp_size)
        self._rollout_stale = False
        return n

    def prepare_for_rollout(self):
        self.prepare_actor_onloaded()
        self.sync_rollout_weights()
        self.rollout_model.eval()

    @torch.no_grad()
    def rollout(self, prompts: list[list[int]], params: SamplingParams, eos_token_ids=(), max_new_tokens: int = 16,
                max_running: int | None = None, progress_interval_s: float | None = None,
                gather_tp: bool = False, stream_ids: list[int] | None = None) -> RolloutOutput:
        """Generate one completion per prompt.  Every rank of a rollout TP group must pass the same
        prompts; with ``gather_tp`` each rank passes only its own prompts, the group's prompts are
        concatenated in rank order, and each rank gets back the results of its own rows.  ``stream_ids`` number the
        random streams of a seeded request (one per prompt; default: the position in ``prompts``): a request that is
        dealt out over data-parallel rows passes each row its prompts' positions in the whole request, so that no
        two of its samples share a stream."""
        self.prepare_for_rollout()
        rctx = self.rollout_ctx
        lo, hi = 0, len(prompts)
        if gather_tp and rctx.tp_size > 1:
            import torch.distributed as dist

            parts: list = [None] * rctx.tp_size
            dist.all_gather_object(parts, (prompts, stream_ids), group=rctx.tp_group)
            lo = sum(len(x[0]) for x in parts[:rctx.tp_rank])
            hi = lo + len(prompts)
            prompts = [row for part in parts for row in part[0]]
            stream_ids = [i for part in parts for i in part[1]] if all(part[1] is not None for part in parts) else None
            max_running = (max_running or self.config.max_running_seqs) * rctx.tp_size
        longest = max((len(p) for p in prompts), default=1) + max_new_tokens
        need_len = (longest + 63) // 64 * 64
        slots = min(max_running or self.config.max_running_seqs, max(len(prompts), 1))
        if rctx.ep_size > 1 and rctx.ep_runtime is not None:
            # expert parallel: the ranks' engines step together and share graph shapes, so they are sized alike
            slots, need_len = rctx.ep_runtime.agree_max([slots, need_len])
        interval = self.config.decode_progress_interval_s if progress_interval_s is None else progress_interval_s
        with use_context(rctx):
            eng = self.inference_engine(slots, need_len)
            with trace_range("rollout"):
                out = eng.generate(prompts, params, eos_token_ids, max_new_tokens, progress_interval_s=interval,
                                   stream_ids=stream_ids)
        if (lo, hi) != (0, len(prompts)):
            out = RolloutOutput(tokens=out.tokens[lo:hi], logprobs=out.logprobs[lo:hi],
                                finish_reasons=out.finish_reasons[lo:hi], stats=out.stats)
        return out

    # ------------------------------------------------------------------ train
    def train(self, packs: list, gradient_accumulation_steps: int | None = None) -> list[dict]:
        self.prepare_for_train()
        self._rollout_stale = True
        with trace_range("train"):
            return self.training_manager().train(packs, gradient_accumulation_steps)

    # ---------------------------------------------------------- GPU residency
    def prepare_for_train(self):
        self.prepare_actor_onloaded()
        if self.infer is not None and not self.config.runtime.keep_rollout_state:
            self.infer.drop_kv_cache()

    def prepare_actor_onloaded(self):
        if not self._actor_on_device:
            with trace_range("offload/onload_actor"):
                self.model.onload_train_weights(self.device)
                if self.trainer is not None:
                    self.trainer.optimizer.onload_state(self.device)
            self._actor_on_device = True

    def prepare_actor_offloaded(self):
        """Move actor weights and optimizer state to the host so another role can use the GPU."""
        if self._actor_on_device:
            if self.infer is not None:
                self.infer.drop_kv_cache()
            if self.trainer is not None:
                self.trainer.optimizer.offload_state()
            self.model.offload_train_weights()
            self._actor_on_device = False
            if self.device.type == "cuda":
                torch.cuda.empty_cache()

    def close(self) -> None:
        """Release what other ranks have mapped (symmetric heaps) after a group barrier; the worker is unusable
        afterwards.  Every rank of the job must call it."""
        if self.infer is not None:
            self.infer._graphs.clear()
        if self.tp_comm is not None:
            from ..parallel import symm

            symm._COMMS.pop(id(self.rollout_ctx), None)
            self.tp_comm.close()
            self.tp_comm = None
        opt = getattr(self.trainer, "optimizer", None)
        if opt is not None and getattr(opt, "grad_comm", None) is not None:
            opt.grad_comm.close()
            opt.grad_comm = None
        ctx = get_context()
        if ctx.ep_runtime is not None:
            ctx.ep_runtime.close()       # expert-parallel heaps (the peers have them mapped)

    def role_manager(self):
        if self.roles is None:
            from .roles import RoleManager

            self.roles = RoleManager(self)
        return self.roles

    def probe_rollout_cache(self, max_running_seqs: int, max_cache_len: int) -> float:
        """Allocate the KV cache (and capture the largest decode graph) for the given rollout shape and
        report the resulting peak memory fraction; used by the auto-tuner."""
        self.prepare_for_rollout()
        if self.device.type == "cuda":
            torch.cuda.reset_peak_memory_stats(self.device)
        with use_context(self.rollout_ctx):
            eng = self.inference_engine(max_running_seqs, (max_cache_len + 63) // 64 * 64)
            eng.ensure_kv_cache()
        return self.peak_memory_fraction()

    def model_info(self) -> dict:
        mc = self.config.model
        return {"model_type": mc.model_type, "vocab_size": mc.vocab_size, "hidden_size": mc.hidden_size,
                "num_hidden_layers": mc.num_hidden_layers, "max_position_embeddings": mc.max_position_embeddings,
                "parameters": sum(p.numel() for p in self.model.parameters()), "tp_size": self.ctx.tp_size,
                "dp_size": self.ctx.dp_size}

    def save_checkpoint(self, path: str) -> None:
        with trace_range("checkpoint/save_weights"):
            self.adapter.save_weights(self.model, path, self.config.model, source_path=self.config.model_path)
        if os.environ.get("ARENO_SAVE_OPTIMIZER", "0") == "1" and self.trainer is not None:
            self.save_training_state(path)

    # Side-car next to the Hugging Face files (an extension: the reference resumes weights only,
    # ``areno/engine/optim/adamw_fp32_master.py:155-237`` has state dicts that nothing calls).  Every rank writes
    # its own optimizer shards; ``state.json`` carries the step counters and the layout they belong to.
    def save_training_state(self, path: str) -> None:
        from safetensors.torch import save_file

        mgr = self.training_manager()
        state = mgr.optimizer.state_dict()
        folder = os.path.join(path, "areno_state")
        os.makedirs(folder, exist_ok=True)
        tensors = {}
        for i, bucket in enumerate(state["buckets"]):
            for key, t in bucket.items():
                if t is not None:
                    tensors[f"bucket{i}.{key}"] = t.contiguous()
        ctx = self.ctx
        save_file(tensors, os.path.join(folder, f"optimizer-rank{ctx.rank:05d}-of-{ctx.world_size:05d}.safetensors"))
        if ctx.rank == 0:
            with open(os.path.join(folder, "state.json"), "w") as f:
                json.dump({"global_step": mgr.global_step, "optimizer_step": state["step"], "dp_size": state["dp_size"],
                           "tp_size": ctx.tp_size, "ep_size": ctx.ep_size, "world_size": ctx.world_size,
                           "adam_8bit": bool(state["adam_8bit"]),
                           "num_buckets": len(state["buckets"])}, f, indent=2)

    def load_training_state(self, path: str) -> bool:
        """Restore optimizer shards and step counters written by ``save_training_state``; returns False when the
        folder is absent or was written for another layout (the run then starts from fresh optimizer state)."""
        from safetensors.torch import load_file

        folder = os.path.join(path, "areno_state")
        meta_path = os.path.join(folder, "state.json")
        if not os.path.isfile(meta_path):
            return False
        with open(meta_path) as f:
            meta = json.load(f)
        ctx = self.ctx
        mgr = self.training_manager()
        opt = mgr.optimizer
        shard = os.path.join(folder, f"optimizer-rank{ctx.rank:05d}-of-{ctx.world_size:05d}.safetensors")
        if (meta.get("world_size") != ctx.world_size or meta.get("tp_size") != ctx.tp_size
                or int(meta.get("ep_size", 1)) != ctx.ep_size or meta.get("num_buckets") != len(opt.buckets) or bool(meta.get("adam_8bit")) != bool(opt.cfg.adam_8bit)
                or not os.path.isfile(shard)):
            logger.warning("training state at %s does not match this layout; starting from fresh optimizer state", folder)
            return False
        tensors = load_file(shard)
        buckets = [{k: tensors.get(f"bucket{i}.{k}") for k in ("master", "m", "v", "m_scale", "v_scale")}
                   for i in range(len(opt.buckets))]
        opt.load_state_dict({"step": meta["optimizer_step"], "dp_size": meta["dp_size"], "buckets": buckets})
        mgr.global_step = int(meta["global_step"])
        return True

    def peak_memory_fraction(self) -> float:
        if self.device.type != "cuda":
            return 0.0
        total = torch.cuda.get_device_properties(self.device).total_memory
        return float(torch.cuda.max_memory_allocated(self.device)) / float(total)
