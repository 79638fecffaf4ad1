"""Continuous-batching inference loop with paged KV and CUDA-graph decode.

One ``InferenceEngine`` lives in each rank worker.  The decode step is
``prepare -> model -> sample -> commit`` entirely on the device (see ``csrc/engine_meta.cu``), so it
is replayed from a CUDA graph per batch bucket with no host read-back; the host learns about
finished sequences from an asynchronously copied status snapshot that it polls without blocking.
Admission, chunked prefill and page allocation are planned by the C++ scheduler.

Semantics kept from the reference loop (``areno/engine/inference.py:199-536``): FIFO admission under
``max_running_seqs`` and the page budget, chunked prefill under ``max_prefill_tokens``, the stop
token is kept in the response, finish reasons ``stop | length | cancelled``, rollout log-probs are
raw-logit log-softmax at temperature 1, new requests may join a running session between steps.
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Callable

import numpy as np
import torch
import torch.distributed as dist

from ..models.dense import InferMeta
from ..ops import _lib as klib
from ..ops import attention as attn_ops
from ..ops import sampling as sampling_ops
from ..ops.paged_attention import PAGE
from ..parallel.context import get_context
from ..utils.log import get_logger
from ..utils.tracing import trace_range
from ._runtime import Scheduler

logger = get_logger()

klib.register_signature("areno_decode_prepare", "ppppiiipppp" + "p")
klib.register_signature("areno_decode_commit", "ppppppppppp" + "iip")
klib.register_signature("areno_prefill_commit", "pppppp" + "i" + "pppppppp" + "ip")

FINISH_NAMES = {0: "running", 1: "stop", 2: "length", 3: "cancelled"}

# Debug guard (``ARENO_CHECK_TOKEN_IDS=1``, as ``areno/engine/runtime/common.py:19,143-159``): every sampled token id
# is range-checked when its sequence is collected, so a degenerate sampler fails loudly instead of feeding ids
# outside the vocabulary to the embedding of the next step or to training.
_CHECK_TOKEN_IDS = os.environ.get("ARENO_CHECK_TOKEN_IDS", "0").lower() in {"1", "true", "yes", "on"}


def _check_token_ids(tokens: list[int], vocab_size: int, name: str) -> None:
    if not tokens:
        return
    lo, hi = min(tokens), max(tokens)
    if lo >= 0 and hi < vocab_size:
        return
    bad = [t for t in tokens if t < 0 or t >= vocab_size]
    raise RuntimeError(f"{name} out of vocab range [0, {vocab_size}): min={lo} max={hi} bad_min={min(bad)} "
                       f"bad_max={max(bad)} count={len(bad)} of {len(tokens)}")


@dataclass
class SamplingParams:
    """Engine-level sampling controls (``areno/engine/data/batch.py:27-38`` in the reference)."""

    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_new_tokens: int = 0
    seed: int | None = None
    stop_token_ids: tuple[int, ...] = ()
    suppress_token_ids: tuple[int, ...] = ()
    # accepted for configurations written for the reference, where it asks the engine to look the special ids up; here
    # the caller names the ids to suppress (the SDK backend derives them from the tokenizer)
    suppress_special_tokens: bool = True


@dataclass
class RolloutOutput:
    tokens: list[list[int]] = field(default_factory=list)
    logprobs: list[list[float]] = field(default_factory=list)
    finish_reasons: list[str] = field(default_factory=list)
    prompt_indices: list[int] | None = None
    stats: dict = field(default_factory=dict)

    # Field names of the reference's rollout result (``areno/engine/data/batch.py``), as read-only views.
    @property
    def response_ids(self) -> list[list[int]]:
        return self.tokens

    @property
    def response_logprobs(self) -> list[list[float]]:
        return self.logprobs

    @property
    def finish_reason(self) -> list[str]:
        return self.finish_reasons

    @property
    def metrics(self) -> dict:
        return self.stats


@dataclass
class _Request:
    rid: int
    prompt: list[int]
    max_new: int
    slot: int = -1
    done: bool = False
    tokens: list[int] | None = None
    logprobs: list[float] | None = None
    reason: str = ""
    tag: object = None
    stream: int = -1  # random-stream id keyed into the sampler; defaults to rid
    # tokens generated before the sequence was sent back to the queue for lack of KV pages; on re-admission they
    # are prefilled together with the prompt and the final result is the concatenation
    kept_tokens: list[int] = field(default_factory=list)
    kept_logprobs: list[float] = field(default_factory=list)

    @property
    def context(self) -> list[int]:
        return self.prompt + self.kept_tokens if self.kept_tokens else self.prompt


def _pick_bucket(buckets: list[int], n: int) -> int:
    for b in buckets:
        if b >= n:
            return b
    return buckets[-1]


class InferenceEngine:
    def __init__(self, model, vocab_size: int, device, *, max_slots: int = 64, max_model_len: int = 4096,
                 max_prefill_tokens: int = 16384, kv_fp8: bool = False, num_pages: int | None = None,
                 graph_buckets: list[int] | None = None, eager: bool = False, seed: int = 0,
                 max_new_cap: int = 4096, stream_salt: int = 0):
        self.model = model
        self.vocab = vocab_size
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.max_slots = max_slots
        self.max_model_len = max_model_len
        self.max_pages = (max_model_len + PAGE - 1) // PAGE
        self.max_prefill_tokens = max_prefill_tokens
        self.kv_fp8 = kv_fp8
        # the checked mode validates indices on the host before every launch, which a captured graph cannot do
        self.eager = eager or not self.cuda or klib.BOUNDS_CHECK
        self.seed = seed
        # Engines of different data-parallel rows share the seed (the ranks of one tensor-parallel group must draw
        # identical noise) and number their requests alike, so unseeded calls mix the row's number into their random
        # streams: without it two samples of one prompt that land on different rows would come out identical.
        self.stream_salt = int(stream_salt)
        self.calls = 0
        self.max_out = max_new_cap
        buckets = sorted(set(graph_buckets or [1, 2, 4, 8, 16, 32, 64, 128, 256, 512]))
        self.buckets = [b for b in buckets if b <= max_slots] or [max_slots]
        if self.buckets[-1] < max_slots:
            self.buckets.append(max_slots)
        self.num_pages = num_pages if num_pages is not None else max_slots * self.max_pages
        self._graphs: dict[int, object] = {}
        self._cls_key = None
        self._alloc_state()
        self.sched: Scheduler | None = None
        self._requests: dict[int, _Request] = {}
        self._next_rid = 0
        self._snapshots: list = []
        self.step_count = 0
        self.decode_tokens = 0
        self._peer_waits = False
        self._lockstep = False
        ctx = get_context()
        # expert-parallel models exchange tokens in every forward pass: see step()
        self._ep = ctx.ep_runtime if (ctx.ep_size > 1 and hasattr(model, "ep_idle_forward")) else None
        self._ep_busy = True
        self._ep_expect_prefill = True

    # ------------------------------------------------------------------ state
    def _alloc_state(self):
        dev, s = self.device, self.max_slots
        i32 = dict(dtype=torch.int32, device=dev)
        self.seq_len = torch.zeros(s, **i32)
        self.active = torch.zeros(s, **i32)
        # finish / gen_count / request uid live in one tensor so a status snapshot is a single D2H copy
        self.state = torch.zeros((3, s), **i32)
        self.finish, self.gen_count, self.uid32 = self.state[0], self.state[1], self.state[2]
        self.max_new = torch.zeros(s, **i32)
        self.last_token = torch.zeros(s, dtype=torch.int64, device=dev)
        self.row_uid = torch.zeros(s, dtype=torch.int64, device=dev)
        self.block_table = torch.zeros((s, self.max_pages), **i32)
        self.out_tokens = torch.zeros((s, self.max_out), **i32)
        self.out_logprobs = torch.zeros((s, self.max_out), dtype=torch.float32, device=dev)
        self.g_input_ids = torch.zeros(s, dtype=torch.int64, device=dev)
        self.g_positions = torch.zeros(s, **i32)
        self.g_slot_mapping = torch.full((s,), -1, **i32)
        self.g_attn_lens = torch.zeros(s, **i32)
        self.sampled = torch.zeros(s, dtype=torch.int64, device=dev)
        self.sampled_lp = torch.zeros(s, dtype=torch.float32, device=dev)
        pin = self.cuda
        self.h_block_table = torch.zeros((s, self.max_pages), dtype=torch.int32, pin_memory=pin)
        self.h_out_tokens = torch.zeros((s, self.max_out), dtype=torch.int32, pin_memory=pin)
        self.h_out_logprobs = torch.zeros((s, self.max_out), dtype=torch.float32, pin_memory=pin)
        self.cls = None
        self.params = SamplingParams()

    def ensure_kv_cache(self):
        if hasattr(self.model, "set_max_slots"):
            self.model.set_max_slots(self.max_slots)   # models with per-slot recurrent state
        if getattr(self.model, "_kv_spec", None) != (self.num_pages, self.kv_fp8):
            self.model.allocate_kv_caches(self.num_pages, self.kv_fp8)
            self._graphs.clear()

    def drop_kv_cache(self):
        self.model.clear_kv_caches()
        self._graphs.clear()

    # ---------------------------------------------------------------- session
    def begin(self, params: SamplingParams, eos_token_ids=(), max_new_tokens: int = 16):
        """Start a generation session: fixes the sampling parameters shared by its requests."""
        self.ensure_kv_cache()
        self.params = params
        stop = tuple(int(t) for t in eos_token_ids) + tuple(int(t) for t in params.stop_token_ids)
        key = (tuple(params.suppress_token_ids), tuple(eos_token_ids), tuple(params.stop_token_ids))
        if key != self._cls_key:
            cls = sampling_ops.build_token_classes(self.vocab, params.suppress_token_ids, eos_token_ids)
            for t in params.stop_token_ids:
                if 0 <= int(t) < self.vocab and cls[int(t)] == 0:
                    cls[int(t)] = 3
            new_cls = cls.to(self.device)
            if self.cls is None:
                self.cls = new_cls
            else:
                self.cls.copy_(new_cls)  # same storage: captured graphs keep pointing at it
            self._cls_key = key
        self.stop_ids = set(stop)
        self.default_max_new = max_new_tokens
        self.sched = Scheduler(self.max_slots, self.num_pages, PAGE, self.max_pages, self.max_prefill_tokens)
        self._requests.clear()
        self._snapshots.clear()
        self.active.zero_()
        self.finish.zero_()
        self.calls += 1
        # The per-call seed travels in the high word of each row's random-stream id (device memory), not
        # as a kernel argument: captured decode graphs stay valid from one call to the next.
        self.call_seed = (params.seed if params.seed is not None else
                          (self.seed * 1000003 + self.calls + 0x9E3779B1 * self.stream_salt)) & 0x7FFFFFFF
        self._graph_key = (params.temperature, params.top_k, params.top_p, params.min_new_tokens)
        self.step_count = 0
        self.decode_tokens = 0
        from ..parallel.symm import get_tp_comm

        self._peer_waits = self.cuda and get_tp_comm(get_context()) is not None
        # Ranks of a tensor-parallel group run the same kernels step for step (each decode step contains collectives),
        # so they must take every scheduling decision at the same loop iteration.  Completions are observed through
        # asynchronous snapshots; letting each rank act on a snapshot "when it has arrived" would let one rank launch
        # a step more than its peer.  In lockstep mode the snapshot taken after step t is consumed exactly
        # ``_LOCKSTEP_LAG`` steps later (waiting for it if need be), which is the same iteration on every rank.
        self._lockstep = get_context().tp_size > 1
        if self._ep is not None:
            self._ep_busy = True
            self._ep_expect_prefill = True
            self._peer_waits = self._peer_waits or self.cuda
            with self._ep.pinned(self.max_slots):
                self._ep.comm(1)     # the decode-sized communicator exists before a graph capture could need it

    def add_request(self, prompt: list[int], max_new_tokens: int | None = None, tag=None,
                    stream: int | None = None) -> int:
        """``stream`` selects the sampler's random stream for this row.  Callers that want a seeded
        request to reproduce pass the row's index within the request; by default every request gets a
        fresh stream."""
        rid = self._next_rid
        self._next_rid += 1
        max_new = self.default_max_new if max_new_tokens is None else max_new_tokens
        room = self.max_model_len - len(prompt)
        max_new = max(1, min(max_new, room, self.max_out))
        if len(prompt) >= self.max_model_len:
            raise ValueError(f"prompt of {len(prompt)} tokens does not fit max_model_len={self.max_model_len}")
        self._requests[rid] = _Request(rid, list(prompt), max_new, tag=tag, stream=rid if stream is None else int(stream))
        self.sched.add(rid, len(prompt), max_new)
        return rid

    @property
    def idle(self) -> bool:
        return self.sched is None or (self.sched.num_running == 0 and self.sched.num_waiting == 0)

    # ------------------------------------------------------------------- step
    @torch.no_grad()
    def step(self) -> list[_Request]:
        """One scheduler iteration: poll completions, prefill newly admitted prompts, run one decode
        step.  Returns the requests that completed since the last call.

        Expert parallelism: every forward pass is an exchange among all ranks, whose engines hold different
        requests.  Before a pass the ranks agree (a host all-reduce of a few integers) on whether anybody runs it
        and at which size; a rank without work of its own joins a prefill with an idle pass and a decode step with
        all slots inactive, so that all ranks launch (and capture) the same sequence of exchanges.  The decode
        agreement also carries how much prefill work and how many uncollected requests any rank still has: while
        nobody can prefill, the prefill agreement of the next iteration is skipped, and when nothing is left
        anywhere the loop of run_until_done ends."""
        done = self._poll(block=False)
        entries = self.sched.plan_prefill()
        ep = self._ep
        if ep is not None:
            g_pre = 0
            if self._ep_expect_prefill:
                g_pre = ep.agree_max([sum(int(e[3]) for e in entries) if entries else 0])[0]
            elif entries:
                raise RuntimeError("expert parallel: prefill work appeared although the last agreement saw none")
            if g_pre > 0:
                with trace_range("rollout/prefill"), ep.pinned(g_pre):
                    if entries:
                        self._run_prefill(entries)
                    else:
                        self.model.ep_idle_forward()
        elif entries:
            with trace_range("rollout/prefill"):
                self._run_prefill(entries)
        updates = None
        had_decoding = self.sched.num_decoding > 0
        if had_decoding:
            while updates is None:
                try:
                    updates = self.sched.reserve_decode(1)
                except MemoryError as exc:
                    # nothing was allocated; make room and ask again (each round frees at least one sequence)
                    done += self._preempt(int(exc.args[0]))
                    if self.sched.num_decoding == 0:
                        updates = []
        decoding = self.sched.num_decoding > 0
        bucket = _pick_bucket(self.buckets, self.sched.active_extent) if decoding else 0
        ctx_cap = self._context_bucket(self.sched.max_seq_len + 1) if decoding else 0
        run_decode = decoding
        if ep is not None:
            sched = self.sched
            prefill_work = sched.num_waiting + max(sched.num_running - sched.num_decoding, 0)
            pending = sched.num_waiting + sched.num_running
            g_dec, bucket, ctx_cap, g_prefill, g_pending = ep.agree_max([int(decoding), bucket, ctx_cap, prefill_work,
                                                                          pending])
            run_decode = bool(g_dec)
            self._ep_expect_prefill = g_prefill > 0
            self._ep_busy = g_pending > 0
        if run_decode:
            if updates:
                self._push_block_updates(updates)
            with trace_range("rollout/decode_step"):
                if ep is not None:
                    with ep.pinned(self.max_slots):
                        self._decode(bucket, ctx_cap)
                else:
                    self._decode(bucket, ctx_cap)
            if decoding:
                self.sched.advance(1)
                self.step_count += 1
                self._snapshot()
                if self._peer_waits and self.step_count % 256 == 0:
                    # kernels that wait on other GPUs report a wait that ran out through the status word: look at
                    # it regularly, not only once the rollout is over
                    klib.check_status(self.device)
        elif not entries and not had_decoding and not self.idle:
            if not self._snapshots:
                self._snapshot()
            with trace_range("rollout/wait_results"):
                done += self._poll(block=True)
        return done

    def run_until_done(self, progress_interval_s: float = 0.0, on_finished: Callable | None = None) -> None:
        t_last = time.time()
        tok_last = 0
        while self._ep is not None or not self.idle:
            if self._ep is not None and not self._ep_busy:
                break             # expert parallel: the loop ends when no rank has work left (agreed in step())
            for req in self.step():
                if on_finished is not None:
                    on_finished(req)
            if progress_interval_s > 0 and time.time() - t_last >= progress_interval_s:
                now = time.time()
                rate = (self.decode_tokens - tok_last) / max(now - t_last, 1e-9)
                ctx = get_context()
                if ctx.tp_rank == 0:      # one line per data-parallel row: the ranks of a TP group decode the same batch
                    logger.info("decode progress row=%d/%d running=%d waiting=%d steps=%d decode_tok_s=%.1f cuda_graph=%s",
                                ctx.dp_rank, ctx.dp_size, self.sched.num_running, self.sched.num_waiting, self.step_count,
                                rate, not self.eager)
                t_last, tok_last = now, self.decode_tokens
        for req in self._poll(block=True, drain=True):
            if on_finished is not None:
                on_finished(req)
        if self.device.type == "cuda":
            klib.check_status(self.device)   # bounded waits that ran out during this rollout surface here

    def generate(self, prompts: list[list[int]], params: SamplingParams, eos_token_ids=(), max_new_tokens: int = 16,
                 progress_interval_s: float = 0.0, stream_ids: list[int] | None = None) -> RolloutOutput:
        """Blocking helper: generate one completion per prompt, results in prompt order.  With a seed the rows draw
        from random streams numbered by ``stream_ids`` (default: their position in ``prompts``)."""
        self.begin(params, eos_token_ids, max_new_tokens)
        seeded = params.seed is not None
        if stream_ids is not None and len(stream_ids) != len(prompts):
            raise ValueError("stream_ids must name one random stream per prompt")
        streams = list(range(len(prompts))) if stream_ids is None else [int(i) for i in stream_ids]
        rids = [self.add_request(p, stream=streams[i] if seeded else None) for i, p in enumerate(prompts)]
        t0 = time.time()
        self.run_until_done(progress_interval_s)
        reqs = [self._requests[r] for r in rids]
        out = RolloutOutput(tokens=[r.tokens or [] for r in reqs], logprobs=[r.logprobs or [] for r in reqs],
                            finish_reasons=[r.reason for r in reqs])
        out.stats = {"decode_steps": self.step_count, "wall_s": time.time() - t0}
        return out

    def cancel_all(self):
        """Mark every running sequence cancelled and drop waiting ones."""
        self.sched.clear_waiting()
        running = (self.active > 0)
        self.finish.masked_fill_(running, 3)
        self.active.zero_()
        self._snapshot()
        for rid, req in self._requests.items():
            if req.slot < 0 and not req.done:
                req.done, req.tokens, req.logprobs, req.reason = True, [], [], "cancelled"

    # ---------------------------------------------------------------- prefill
    def _run_prefill(self, entries):
        dev = self.device
        ids, pos, slots_map, q_lens, k_lens = [], [], [], [], []
        logit_rows, fin_slots, fin_prompt, fin_budget, fin_uid, fin_stream = [], [], [], [], [], []
        hist_slots = []
        seq_slots, seq_fresh = [], []
        has_history = False
        row = 0
        for slot, rid, start, length, last in entries:
            seq_slots.append(slot)
            seq_fresh.append(1 if start == 0 else 0)
            req = self._requests[rid]
            req.slot = slot
            pages = self.sched.slot_pages(slot)
            self.h_block_table[slot, : len(pages)] = torch.tensor(pages, dtype=torch.int32)
            chunk = req.context[start:start + length]
            ids.extend(chunk)
            p = np.arange(start, start + length)
            pos.append(p)
            pg = np.asarray(pages, dtype=np.int64)
            slots_map.append(pg[p // PAGE] * PAGE + p % PAGE)
            q_lens.append(length)
            k_lens.append(start + length)
            if start > 0:
                has_history = True
            allp = np.arange(0, start + length)
            hist_slots.append(pg[allp // PAGE] * PAGE + allp % PAGE)
            row += length
            if last:
                logit_rows.append(row - 1)
                fin_slots.append(slot)
                fin_prompt.append(len(req.context))
                fin_budget.append(req.max_new - len(req.kept_tokens))
                fin_uid.append(rid)
                fin_stream.append(req.stream)
        touched = sorted({e[0] for e in entries})
        lo, hi = touched[0], touched[-1] + 1
        self.block_table[lo:hi].copy_(self.h_block_table[lo:hi], non_blocking=True)
        ids_t = torch.tensor(ids, dtype=torch.int64)
        pos_t = torch.from_numpy(np.concatenate(pos).astype(np.int32))
        slot_t = torch.from_numpy(np.concatenate(slots_map).astype(np.int32))
        if self.cuda:
            ids_t, pos_t, slot_t = (t.pin_memory().to(dev, non_blocking=True) for t in (ids_t, pos_t, slot_t))
        meta = InferMeta(mode="prefill", slot_mapping=slot_t,
                         varlen=attn_ops.build_varlen_meta(q_lens, k_lens, device=dev), has_history=has_history,
                         seq_slots=torch.tensor(seq_slots, dtype=torch.int32, device=dev),
                         seq_fresh=torch.tensor(seq_fresh, dtype=torch.int32, device=dev))
        if has_history:
            meta.history = torch.from_numpy(np.concatenate(hist_slots)).to(dev)
        if logit_rows:
            meta.logit_rows = torch.tensor(logit_rows, dtype=torch.int64, device=dev)
        else:
            meta.logit_rows = torch.zeros(0, dtype=torch.int64, device=dev)
        out = self.model(ids_t, pos_t, meta)
        n = len(logit_rows)
        if n == 0:
            return
        uid = torch.tensor(fin_uid, dtype=torch.int64, device=dev)
        slots_t = torch.tensor(fin_slots, dtype=torch.int32, device=dev)
        stream = torch.tensor([(self.call_seed << 32) | (int(x) & 0xFFFFFFFF) for x in fin_stream], dtype=torch.int64,
                              device=dev)
        self.row_uid[slots_t.long()] = stream
        self.uid32[slots_t.long()] = (uid & 0x7FFFFFFF).to(torch.int32)
        zero_gen = torch.zeros(n, dtype=torch.int32, device=dev)
        tok, lp = self._sample(out.logits_shard, zero_gen, stream)
        prompt_t = torch.tensor(fin_prompt, dtype=torch.int32, device=dev)
        budget_t = torch.tensor(fin_budget, dtype=torch.int32, device=dev)
        if self.cuda:
            klib.call("areno_prefill_commit", tok.data_ptr(), lp.data_ptr(), self.cls.data_ptr(), slots_t.data_ptr(),
                      prompt_t.data_ptr(), budget_t.data_ptr(), n, self.seq_len.data_ptr(), self.active.data_ptr(),
                      self.last_token.data_ptr(), self.gen_count.data_ptr(), self.max_new.data_ptr(),
                      self.finish.data_ptr(), self.out_tokens.data_ptr(), self.out_logprobs.data_ptr(), self.max_out,
                      klib.stream())
        else:
            self._prefill_commit_cpu(tok, lp, fin_slots, fin_prompt, fin_budget)
        self._snapshot()

    def _prefill_commit_cpu(self, tok, lp, slots, prompts, budgets):
        for j, s in enumerate(slots):
            t = int(tok[j])
            self.out_tokens[s, 0] = t
            self.out_logprobs[s, 0] = lp[j]
            self.gen_count[s] = 1
            self.max_new[s] = budgets[j]
            self.seq_len[s] = prompts[j]
            self.last_token[s] = t
            c = int(self.cls[t])
            if c in (2, 3):
                self.finish[s], self.active[s] = 1, 0
            elif budgets[j] <= 1:
                self.finish[s], self.active[s] = 2, 0
            else:
                self.finish[s], self.active[s] = 0, 1

    # ----------------------------------------------------------------- sample
    def _sample(self, logits, gen_count, row_uid, out_token=None, out_logprob=None):
        p = self.params
        ctx = get_context()
        lm = self.model.lm_head
        valid = lm.valid_local
        view = logits[:, :valid]
        if ctx.tp_size == 1:
            return sampling_ops.sample(view, p.temperature, p.top_k, p.top_p, cls=self.cls, gen_count=gen_count,
                                       min_new=p.min_new_tokens, seed=self.seed, row_uid=row_uid,
                                       out_token=out_token, out_logprob=out_logprob)
        if (p.top_k > 0 or p.top_p < 1.0) and p.temperature > 0:
            # truncated sampling needs the whole distribution on one rank
            full = torch.empty((ctx.tp_size * view.shape[0], view.shape[1]), dtype=view.dtype, device=view.device)
            dist.all_gather_into_tensor(full, view.contiguous(), group=ctx.tp_group)
            full = full.view(ctx.tp_size, *view.shape).permute(1, 0, 2).reshape(view.shape[0], -1)[:, : self.vocab].contiguous()
            return sampling_ops.sample(full, p.temperature, p.top_k, p.top_p, cls=self.cls, gen_count=gen_count,
                                       min_new=p.min_new_tokens, seed=self.seed, row_uid=row_uid,
                                       out_token=out_token, out_logprob=out_logprob)
        part = torch.empty((view.shape[0], 6), dtype=torch.float32, device=view.device)
        sampling_ops.sample(view, p.temperature, p.top_k, p.top_p, cls=self.cls, gen_count=gen_count,
                            min_new=p.min_new_tokens, seed=self.seed, row_uid=row_uid,
                            vocab_start=lm.vocab_start, part=part)
        parts = torch.empty((ctx.tp_size * part.shape[0], 6), dtype=torch.float32, device=view.device)
        dist.all_gather_into_tensor(parts, part, group=ctx.tp_group)
        tok, lp = sampling_ops.combine_shards(parts.view(ctx.tp_size, *part.shape))
        if out_token is not None:
            out_token.copy_(tok)
            out_logprob.copy_(lp)
            return out_token, out_logprob
        return tok, lp

    # ----------------------------------------------------------------- decode
    def _context_bucket(self, tokens: int) -> int:
        """Static bound on the context length of a decode step: the next power-of-two number of pages.  The
        attention launch (number of KV splits) is sized for this bound instead of the model length, and a
        captured graph is kept per bound."""
        pages = max(1, (tokens + PAGE - 1) // PAGE)
        cap = 4
        while cap < pages:
            cap *= 2
        return min(cap * PAGE, self.max_pages * PAGE)

    def _decode_body(self, b: int, ctx_cap: int | None = None):
        if self.cuda:
            klib.call("areno_decode_prepare", self.seq_len.data_ptr(), self.active.data_ptr(),
                      self.last_token.data_ptr(), self.block_table.data_ptr(), self.max_pages, PAGE, b,
                      self.g_input_ids.data_ptr(), self.g_positions.data_ptr(), self.g_slot_mapping.data_ptr(),
                      self.g_attn_lens.data_ptr(), klib.stream())
        else:
            act = self.active[:b] > 0
            pos = self.seq_len[:b]
            page = self.block_table[:b].gather(1, (pos // PAGE).long().clamp(max=self.max_pages - 1)[:, None])[:, 0]
            self.g_positions[:b] = torch.where(act, pos, torch.zeros_like(pos))
            self.g_slot_mapping[:b] = torch.where(act, page * PAGE + pos % PAGE, torch.full_like(pos, -1))
            self.g_attn_lens[:b] = torch.where(act, pos + 1, torch.zeros_like(pos))
            self.g_input_ids[:b] = torch.where(act, self.last_token[:b], torch.zeros_like(self.last_token[:b]))
        meta = InferMeta(mode="decode", slot_mapping=self.g_slot_mapping[:b], block_table=self.block_table[:b],
                         seq_lens=self.g_attn_lens[:b], max_context=ctx_cap or self.max_model_len)
        out = self.model(self.g_input_ids[:b], self.g_positions[:b], meta)
        self._sample(out.logits_shard, self.gen_count[:b], self.row_uid[:b], self.sampled[:b], self.sampled_lp[:b])
        if self.cuda:
            klib.call("areno_decode_commit", self.sampled.data_ptr(), self.sampled_lp.data_ptr(), self.cls.data_ptr(),
                      self.seq_len.data_ptr(), self.active.data_ptr(), self.last_token.data_ptr(),
                      self.gen_count.data_ptr(), self.max_new.data_ptr(), self.finish.data_ptr(),
                      self.out_tokens.data_ptr(), self.out_logprobs.data_ptr(), self.max_out, b, klib.stream())
        else:
            for i in range(b):
                if not int(self.active[i]):
                    continue
                t, g = int(self.sampled[i]), int(self.gen_count[i])
                self.out_tokens[i, g] = t
                self.out_logprobs[i, g] = self.sampled_lp[i]
                self.gen_count[i] = g + 1
                self.seq_len[i] += 1
                self.last_token[i] = t
                c = int(self.cls[t])
                if c in (2, 3):
                    self.finish[i], self.active[i] = 1, 0
                elif g + 1 >= int(self.max_new[i]):
                    self.finish[i], self.active[i] = 2, 0

    def _decode(self, b: int, ctx_cap: int | None = None):
        self.decode_tokens += self.sched.num_decoding
        if self.eager:
            self._decode_body(b, ctx_cap)
            return
        key = (b, ctx_cap, self._graph_key)
        entry = self._graphs.get(key)
        if entry is None:
            before = klib.launch_count
            graph = self._capture(b, ctx_cap)
            entry = (graph, (klib.launch_count - before) // 3)  # two warm-up passes + the captured one
            self._graphs[key] = entry
        entry[0].replay()
        klib.launch_count += entry[1]

    def _capture(self, b: int, ctx_cap: int | None = None):
        # Warm up on a side stream (allocations, lazy module state), then capture.  The warm-up and
        # the capture pass run real decode steps on the slot state, so that state is saved and
        # restored around them.
        saved = [t.clone() for t in (self.seq_len, self.active, self.last_token, self.gen_count, self.finish,
                                     self.out_tokens[:, :2], self.out_logprobs[:, :2])]
        active_real = self.active.clone()
        self.active.zero_()          # warm-up steps touch no KV slot and commit nothing
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._decode_body(b, ctx_cap)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._decode_body(b, ctx_cap)
        self.active.copy_(active_real)
        for dst, src in zip((self.seq_len, self.active, self.last_token, self.gen_count, self.finish), saved[:5]):
            dst.copy_(src)
        self.out_tokens[:, :2].copy_(saved[5])
        self.out_logprobs[:, :2].copy_(saved[6])
        return graph

    # ------------------------------------------------------------ bookkeeping
    def _push_block_updates(self, updates):
        for slot, idx, page in updates:
            self.h_block_table[slot, idx] = page
        slots = sorted({u[0] for u in updates})
        lo, hi = slots[0], slots[-1] + 1
        self.block_table[lo:hi].copy_(self.h_block_table[lo:hi], non_blocking=True)

    def _snapshot(self):
        """Queue an async copy of the (finish, gen_count, uid) status rows for the host to poll."""
        if not self.cuda:
            self._snapshots.append((self.state.clone(), None))
            return
        # ring of pinned buffers (pinned allocation is far too slow to do per step)
        if not hasattr(self, "_snap_ring"):
            self._snap_ring = [torch.empty((3, self.max_slots), dtype=torch.int32, pin_memory=True) for _ in range(8)]
            self._snap_events = [torch.cuda.Event() for _ in range(8)]
            self._snap_next = 0
        while len(self._snapshots) >= 6 and not self._lockstep:
            # bound how far the device may run ahead of the host; a newer snapshot supersedes older ones
            self._snapshots[0][1].synchronize()
            if len(self._snapshots) >= 7:
                self._snapshots.pop(0)
            else:
                break
        if self._lockstep and len(self._snapshots) >= len(self._snap_ring):
            # cannot happen while every step consumes what exceeds the lag; a ring slot must never be reused while queued
            raise RuntimeError("snapshot ring exhausted in lockstep mode")
        i = self._snap_next
        self._snap_next = (i + 1) % len(self._snap_ring)
        host = self._snap_ring[i]
        host.copy_(self.state, non_blocking=True)
        ev = self._snap_events[i]
        ev.record()
        self._snapshots.append((host, ev))

    def _poll(self, block: bool, drain: bool = False) -> list[_Request]:
        if self._lockstep:
            return self._poll_lockstep(block, drain)
        done: list[_Request] = []
        latest = None
        while self._snapshots:
            host, ev = self._snapshots[0]
            if ev is not None and not ev.query():
                if not (block or drain):
                    break
                ev.synchronize()
            latest = host
            self._snapshots.pop(0)
            if block and not drain:
                block = False
        if latest is None:
            return done
        return done + self._collect(latest)

    _LOCKSTEP_LAG = 4

    def _poll_lockstep(self, block: bool, drain: bool) -> list[_Request]:
        """Consume snapshots strictly in order and at a fixed distance behind the launches: non-blocking calls take
        the oldest snapshot only once more than ``_LOCKSTEP_LAG`` are queued, ``block`` takes exactly the oldest one,
        ``drain`` takes them all.  Which snapshot is looked at therefore depends on the iteration count alone."""
        done: list[_Request] = []
        while self._snapshots:
            if not (drain or block or len(self._snapshots) > self._LOCKSTEP_LAG):
                break
            host, ev = self._snapshots.pop(0)
            if ev is not None:
                ev.synchronize()
            done += self._collect(host)
            if block and not drain:
                break
        return done

    def _collect(self, latest) -> list[_Request]:
        """Hand out the sequences that ``latest`` (a host copy of the status rows) shows as finished."""
        done: list[_Request] = []
        fin, gen, uid = latest[0], latest[1], latest[2]
        finished_slots = []
        for slot in range(self.max_slots):
            f = int(fin[slot])
            if f == 0:
                continue
            rid = self.sched.slot_request(slot)
            if rid < 0:
                continue
            req = self._requests.get(rid)
            if req is None or req.done or req.slot != slot or int(uid[slot]) != (rid & 0x7FFFFFFF):
                continue
            finished_slots.append((slot, req, f, int(gen[slot])))
        if not finished_slots:
            return done
        for slot, req, f, g in finished_slots:
            self.h_out_tokens[slot, :g].copy_(self.out_tokens[slot, :g], non_blocking=True)
            self.h_out_logprobs[slot, :g].copy_(self.out_logprobs[slot, :g], non_blocking=True)
        if self.cuda:
            torch.cuda.current_stream().synchronize()
        for slot, req, f, g in finished_slots:
            req.tokens = req.kept_tokens + self.h_out_tokens[slot, :g].tolist()
            req.logprobs = req.kept_logprobs + self.h_out_logprobs[slot, :g].tolist()
            if _CHECK_TOKEN_IDS:
                _check_token_ids(req.tokens, self.vocab, f"sampled tokens of request {req.rid}")
            req.reason = FINISH_NAMES.get(f, "stop")
            req.done = True
            self.finish[slot] = 0
            self.sched.finish(slot)
            done.append(req)
        return done

    def _preempt(self, slot: int) -> list[_Request]:
        """Out of KV pages while reserving the next decode step (``slot`` is the first one that did not fit).

        The sequence admitted last goes back to the head of the waiting queue with what it has generated so far:
        its pages are freed now, and when pages are available again it is prefilled as prompt + generated tokens and
        carries on, so the caller still gets a complete response.  (The reference raises "paged KV cache exhausted
        during decode", ``areno/engine/data/rollout_state.py:212-225``.)  Only when a single sequence is decoding,
        so that evicting it would make room for nobody, is it finished early with reason ``length``.  Returns the
        requests that completed while making room."""
        victim = self.sched.preempt_victim()
        if self.cuda:
            torch.cuda.current_stream().synchronize()   # the device state below is final for every launched step
        if victim < 0:
            self.finish[slot] = 2
            self.active[slot] = 0
            self._snapshot()
            return self._poll(block=True, drain=True)
        rid = self.sched.slot_request(victim)
        req = self._requests.get(rid)
        fin, g = int(self.finish[victim]), int(self.gen_count[victim])
        if req is None or fin != 0:
            # it finished in a step the host has not seen yet: collecting it frees its pages
            self._snapshot()
            return self._poll(block=True, drain=True)
        req.kept_tokens = req.kept_tokens + self.out_tokens[victim, :g].tolist()
        req.kept_logprobs = req.kept_logprobs + self.out_logprobs[victim, :g].tolist()
        self.active[victim] = 0
        self.gen_count[victim] = 0
        req.slot = -1
        self._snapshots.clear()     # older snapshots describe the evicted occupant of this slot
        self.sched.requeue(victim, len(req.context), req.max_new - len(req.kept_tokens))
        logger.info("KV pages exhausted: request %d re-queued after %d generated tokens", rid, len(req.kept_tokens))
        return []
