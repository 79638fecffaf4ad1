"""The engine coordinator against a scripted cluster, on the CPU: how prompts, score rows and training packs are dealt
out over the data-parallel rows, which rank's answer counts for a row, and how the answers come back in the caller's
order.  Behaviours follow the reference's ``tests/test_runtime_utils_cpu.py`` and the coordinator half of its
``tests/test_inference_scheduler_cpu.py``."""

from __future__ import annotations

import asyncio

import pytest
import torch

from areno_b200.engine import api as engine_api
from areno_b200.engine.api import (ArenoEngine, dp_rank0_results, merge_rollouts_in_input_order, split_list_by_dp)
from areno_b200.engine.config import EngineConfig
from areno_b200.engine.inference import RolloutOutput, SamplingParams
from areno_b200.engine.protocol import Op, RolloutPayload
from areno_b200.engine.training import merge_train_stats, split_data_pack_by_dp
from tests.helpers import tiny_config


class ScriptedCluster:
    """Answers like ``world`` ranks would: ``handler(op, payload, rank, dp_rank, tp_rank)`` per rank."""

    is_spmd = False

    def __init__(self, config, handler):
        self.config, self.handler, self.calls = config, handler, []

    def _run(self, op, payload, result_ranks=None):
        self.calls.append((op, payload, result_ranks))
        tp = self.config.rollout_tp if op in (Op.INFER_ROLLOUT, Op.PROBE_ROLLOUT_CACHE) else self.config.tp_size
        out = []
        for rank in range(self.config.world_size):
            if result_ranks is not None and rank not in result_ranks:
                continue
            out.append(self.handler(op, payload, rank, rank // tp, rank % tp))
        return out

    def call(self, op, payload=None, timeout=None, **kw):
        return self._run(op, payload)

    async def call_async(self, op, payload=None, result_ranks=None):
        return self._run(op, payload, result_ranks)

    def close(self):
        pass


def _engine(handler, monkeypatch, **cfg):
    config = EngineConfig(model=tiny_config(), **cfg)
    holder = {}

    def fake_make_cluster(c, launcher, worker):
        holder["cluster"] = ScriptedCluster(c, handler)
        return holder["cluster"]

    monkeypatch.setattr(engine_api, "make_cluster", fake_make_cluster)
    eng = ArenoEngine(config)
    return eng, holder["cluster"]


# ------------------------------------------------------------------------------------------------ plain helpers

def test_lists_are_dealt_round_robin():
    assert split_list_by_dp(list(range(7)), 3) == [[0, 3, 6], [1, 4], [2, 5]]
    assert split_list_by_dp([], 2) == [[], []] and split_list_by_dp([1], 1) == [[1]]


def test_one_answer_per_data_parallel_row():
    answers = [f"r{r}" for r in range(8)]
    assert dp_rank0_results(answers, tp_size=2, dp_size=4) == ["r0", "r2", "r4", "r6"]
    assert dp_rank0_results(answers, tp_size=8, dp_size=1) == ["r0"]
    assert dp_rank0_results(answers, tp_size=1, dp_size=8) == answers


def test_packs_are_split_by_stride_and_small_batches_replicated():
    pack = {"input_ids": torch.arange(12).view(6, 2), "lengths": torch.arange(6), "names": list("abcdef"),
            "scalar": 3, "table": torch.zeros(4, 4)}
    shards = split_data_pack_by_dp(pack, 3)
    assert [s["lengths"].tolist() for s in shards] == [[0, 3], [1, 4], [2, 5]]
    assert shards[1]["names"] == ["b", "e"] and shards[2]["input_ids"].tolist() == [[4, 5], [10, 11]]
    assert all(s["scalar"] == 3 and s["table"] is pack["table"] for s in shards)
    tiny = {"input_ids": torch.zeros(2, 3)}
    assert all(s is tiny for s in split_data_pack_by_dp(tiny, 4)) and len(split_data_pack_by_dp(tiny, 4)) == 4
    assert split_data_pack_by_dp({"x": 1}, 2) == [{"x": 1}, {"x": 1}]


def test_train_statistics_average_over_rows():
    a = {"loss": 1.0, "step": 4, "metrics": {"kl": 0.2, "clip": 1, "name": "a"}}
    b = {"loss": 3.0, "step": 4, "metrics": {"kl": 0.4, "clip": 3, "name": "b"}}
    merged = merge_train_stats([a, None, b, {}])
    assert merged["loss"] == 2.0 and merged["step"] == 4
    assert merged["metrics"] == {"kl": pytest.approx(0.3), "clip": 2.0, "name": "a"}
    assert merge_train_stats([]) == {} and merge_train_stats([None]) == {}


def test_rollout_shares_return_to_input_positions_with_merged_statistics():
    a = RolloutOutput(tokens=[[1], [3]], logprobs=[[-1.0], [-3.0]], finish_reasons=["stop", "length"], prompt_indices=[0, 2],
                      stats={"decode_steps": 5, "wall_s": 1.5, "generated": 2, "bucket": "b64"})
    b = RolloutOutput(tokens=[[2]], logprobs=[[-2.0]], finish_reasons=["stop"], prompt_indices=[1],
                      stats={"decode_steps": 7, "wall_s": 1.0, "generated": 1})
    merged = merge_rollouts_in_input_order([a, None, b], 3)
    assert merged.tokens == [[1], [2], [3]] and merged.logprobs == [[-1.0], [-2.0], [-3.0]]
    assert merged.finish_reasons == ["stop", "stop", "length"] and merged.prompt_indices == [0, 1, 2]
    assert merged.stats == {"decode_steps": 7, "wall_s": 1.5, "generated": 3, "bucket": "b64"}
    assert merged.response_ids is merged.tokens and merged.finish_reason is merged.finish_reasons
    empty = merge_rollouts_in_input_order([], 2)
    assert empty.tokens == [[], []] and empty.finish_reasons == ["", ""] and empty.stats == {}


# ----------------------------------------------------------------------------------------------------- rollout

def _echo_rollout(op, payload, rank, dp_rank, tp_rank):
    assert op is Op.INFER_ROLLOUT
    prompts, idx = payload.prompts_by_dp[dp_rank], payload.prompt_indices_by_dp[dp_rank]
    mark = 100 * tp_rank                       # only TP rank 0's copy may be used
    return RolloutOutput(tokens=[[p[0] + mark] for p in prompts], logprobs=[[-float(i)] for i in idx],
                         finish_reasons=["stop"] * len(idx), prompt_indices=list(idx), stats={"generated": len(idx)})


def test_rollout_deals_prompts_out_and_merges_in_input_order(monkeypatch):
    eng, cluster = _engine(_echo_rollout, monkeypatch, tp_size=2, dp_size=2)
    prompts = [[10, 1], [11], [12, 1, 1], [13], [14]]
    out = eng.generate_rollout(prompts, max_new_tokens=6, max_running_prompts=5, eos_token_id=2)
    assert out.tokens == [[10], [11], [12], [13], [14]] and out.logprobs == [[-0.0], [-1.0], [-2.0], [-3.0], [-4.0]]
    assert out.stats == {"generated": 5}
    op, payload, _ = cluster.calls[0]
    assert isinstance(payload, RolloutPayload) and payload.prompts_by_dp == [[[10, 1], [12, 1, 1], [14]], [[11], [13]]]
    assert payload.prompt_indices_by_dp == [[0, 2, 4], [1, 3]]
    assert payload.eos_token_ids == (2,) and payload.max_running_seqs == 3          # ceil(5 / 2) per row
    assert payload.max_cache_len == 3 + 6 and payload.max_new_tokens == 6


def test_rollout_argument_checks_and_eos_forms(monkeypatch):
    eng, cluster = _engine(_echo_rollout, monkeypatch)
    with pytest.raises(ValueError, match="non-empty"):
        eng.generate_rollout([], max_new_tokens=4, max_running_prompts=1)
    with pytest.raises(ValueError, match="max_running_prompts"):
        eng.generate_rollout([[1]], max_new_tokens=4, max_running_prompts=0)
    eng.generate_rollout([[1]], max_new_tokens=4, max_running_prompts=1)
    eng.generate_rollout([[1]], max_new_tokens=4, max_running_prompts=1, eos_token_id=[5, 6],
                         sampling_params=SamplingParams(temperature=0.5))
    assert cluster.calls[0][1].eos_token_ids == () and cluster.calls[1][1].eos_token_ids == (5, 6)
    assert cluster.calls[1][1].sampling_params.temperature == 0.5
    with pytest.raises(RuntimeError, match="SPMD launcher"):
        eng.generate_rollout([[1]], max_new_tokens=4, max_running_prompts=1, local=True)


def test_rollout_layout_follows_the_rollout_tp_width(monkeypatch):
    cfg = dict(tp_size=1, dp_size=4, rollout_tp_size=2)
    config_model = tiny_config(num_attention_heads=4, num_key_value_heads=2)
    config = EngineConfig(model=config_model, **cfg)
    monkeypatch.setattr(engine_api, "make_cluster", lambda c, launcher, worker: ScriptedCluster(c, _echo_rollout))
    eng = ArenoEngine(config)
    out = eng.generate_rollout([[1], [2], [3]], max_new_tokens=2, max_running_prompts=4)
    payload = eng.cluster.calls[0][1]
    assert len(payload.prompts_by_dp) == 2 and payload.max_running_seqs == 2        # two rollout rows of two ranks
    assert out.tokens == [[1], [2], [3]]


def test_single_requests_go_to_one_row_each_in_turn(monkeypatch):
    eng, cluster = _engine(_echo_rollout, monkeypatch, tp_size=2, dp_size=3)

    async def run():
        return [await eng.generate_rollout_async([[20 + i]], max_new_tokens=3, max_running_prompts=2) for i in range(4)]

    outs = asyncio.run(run())
    assert [o.tokens for o in outs] == [[[20]], [[21]], [[22]], [[23]]]
    owners = [next(r for r, p in enumerate(c[1].prompts_by_dp) if p) for c in cluster.calls]
    assert owners == [0, 1, 2, 0]
    assert [c[2] for c in cluster.calls] == [{0}, {2}, {4}, {0}]                 # TP rank 0 of the owning row
    assert cluster.calls[0][1].max_running_seqs == 2                              # per-row capacity, not divided again
    with pytest.raises(ValueError, match="non-empty"):
        asyncio.run(eng.generate_rollout_async([], max_new_tokens=3, max_running_prompts=2))


def test_single_request_merge_ignores_rows_without_work(monkeypatch):
    def handler(op, payload, rank, dp_rank, tp_rank):
        out = _echo_rollout(op, payload, rank, dp_rank, tp_rank)
        return out if out.prompt_indices else RolloutOutput(prompt_indices=[])

    eng, cluster = _engine(handler, monkeypatch, tp_size=1, dp_size=2)
    cluster._run_all = cluster._run
    cluster._run = lambda op, payload, result_ranks=None: cluster._run_all(op, payload, None)     # every rank answers
    next(eng._dp_cursor)                                                        # the next owner is row 1
    out = asyncio.run(eng.generate_rollout_async([[7], [8]], max_new_tokens=2, max_running_prompts=1))
    assert out.tokens == [[7], [8]]


def test_request_concurrent_rollout_is_refused_under_expert_parallelism(monkeypatch):
    moe = tiny_config(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64)
    config = EngineConfig(model=moe, tp_size=1, dp_size=2, expert_parallel=True)
    monkeypatch.setattr(engine_api, "make_cluster", lambda c, launcher, worker: ScriptedCluster(c, _echo_rollout))
    eng = ArenoEngine(config)
    with pytest.raises(RuntimeError, match="expert"):
        asyncio.run(eng.generate_rollout_async([[1]], max_new_tokens=2, max_running_prompts=1))


def test_cache_probe_reports_the_tightest_rank(monkeypatch):
    def handler(op, payload, rank, dp_rank, tp_rank):
        assert op is Op.PROBE_ROLLOUT_CACHE and payload.max_running_seqs == 3 and payload.max_cache_len == 48
        return [0.25, None, 0.75, 0.5][rank]

    eng, _ = _engine(handler, monkeypatch, tp_size=1, dp_size=4)
    assert eng.probe_rollout_cache(max_new_tokens=16, max_running_prompts=10, max_prompt_len=32) == 0.75
    with pytest.raises(ValueError):
        eng.probe_rollout_cache(max_new_tokens=0, max_running_prompts=1, max_prompt_len=1)


# --------------------------------------------------------------------------------------------- scoring, training

def test_scores_return_in_row_order_from_strided_shares(monkeypatch):
    def handler(op, payload, rank, dp_rank, tp_rank):
        assert payload.role == "ref" and payload.pad_token_id == 9
        return [[float(sum(r)) + 1000 * tp_rank] for r in payload.rows_by_dp[dp_rank]]

    eng, cluster = _engine(handler, monkeypatch, tp_size=2, dp_size=3)
    rows = [[i, i] for i in range(8)]
    assert eng.score_logprobs("ref", rows, pad_token_id=9, microbatch_size=4) == [[2.0 * i] for i in range(8)]
    assert cluster.calls[0][0] is Op.SCORE_LOGPROBS and cluster.calls[0][1].microbatch_size == 4
    assert cluster.calls[0][1].rows_by_dp[1] == [[1, 1], [4, 4], [7, 7]]
    eng.score_values("ref", rows[:2], pad_token_id=9)
    eng.score_rewards("ref", rows[:2], pad_token_id=9)
    assert [c[0] for c in cluster.calls[1:]] == [Op.SCORE_VALUES, Op.SCORE_REWARDS]


def test_step_averages_each_micro_step_over_the_rows(monkeypatch):
    def handler(op, payload, rank, dp_rank, tp_rank):
        assert op is Op.TRAIN and payload.gradient_accumulation_steps == 2
        return [{"loss": float(dp_rank + 10 * i + 100 * tp_rank), "metrics": {"tokens": shards[dp_rank]["lengths"].sum().item()}}
                for i, shards in enumerate(payload.packs)]

    eng, cluster = _engine(handler, monkeypatch, tp_size=2, dp_size=2)
    packs = [{"input_ids": torch.zeros(4, 3), "lengths": torch.tensor([1, 2, 3, 4])},
             {"input_ids": torch.zeros(2, 3), "lengths": torch.tensor([5, 7])}]
    stats = eng.step(packs, gradient_accumulation_steps=2)
    assert [s["loss"] for s in stats] == [0.5, 10.5]
    assert stats[0]["metrics"]["tokens"] == 5.0 and stats[1]["metrics"]["tokens"] == 6.0
    assert eng.step([]) == [] and len(cluster.calls) == 1


def test_critic_statistics_are_the_mean_over_rows(monkeypatch):
    def handler(op, payload, rank, dp_rank, tp_rank):
        assert (payload.role, payload.cliprange_value, payload.value_loss_coef) == ("critic", 0.3, 0.7)
        return {"value_loss": float(dp_rank), "clipfrac": 0.5} if dp_rank < 2 else {}

    eng, _ = _engine(handler, monkeypatch, tp_size=1, dp_size=3)
    out = eng.train_values("critic", [{"input_ids": torch.zeros(3, 2)}], cliprange_value=0.3, value_loss_coef=0.7)
    assert out == {"value_loss": 0.5, "clipfrac": 0.5}

    eng2, _ = _engine(lambda *a: {}, monkeypatch, tp_size=1, dp_size=2)
    assert eng2.train_values("critic", [{"input_ids": torch.zeros(2, 2)}]) == {}


def test_session_and_housekeeping_calls_reach_every_rank(monkeypatch):
    seen = []

    def handler(op, payload, rank, dp_rank, tp_rank):
        seen.append((op, rank))
        return {"model_type": "qwen2"} if op is Op.MODEL_INFO else None

    eng, cluster = _engine(handler, monkeypatch, tp_size=1, dp_size=2)
    eng.begin_rollout_session()
    asyncio.run(eng.sync_rollout_session_async())
    eng.end_rollout_session()
    eng.ensure_roles({"ref": object()})
    assert eng.save_checkpoint("/tmp/x") == "/tmp/x"
    ops = [c[0] for c in cluster.calls]
    assert ops == [Op.ROLLOUT_SESSION_BEGIN, Op.ROLLOUT_SESSION_SYNC, Op.ROLLOUT_SESSION_END, Op.ENSURE_ROLES,
                   Op.SAVE_CHECKPOINT]
    assert cluster.calls[4][1].path == "/tmp/x" and len(seen) == 10


def test_from_pretrained_needs_a_model_or_a_config(monkeypatch):
    with pytest.raises(ValueError, match="model path or an explicit model_config"):
        ArenoEngine.from_pretrained(None)
    monkeypatch.setattr(engine_api, "make_cluster", lambda c, launcher, worker: ScriptedCluster(c, lambda *a: None))
    eng = ArenoEngine.from_pretrained(None, model_config=tiny_config(), tp_size=2, dp_size=2, max_running_seqs=7, seed=5)
    assert eng.config.dummy_load and eng.config.world_size == 4 and eng.config.max_running_seqs == 7 and eng.config.seed == 5


def test_payloads_are_narrowed_to_what_a_rank_reads():
    from areno_b200.engine.protocol import (CachePayload, ScorePayload, TrainPayload, TrainValuesPayload, narrow_for_rank)

    roll = RolloutPayload([[[1], [2]], [[3]], [[4]]], [[0, 3], [1], [2]], max_new_tokens=4, max_cache_len=9)
    mine = narrow_for_rank(roll, train_dp_rank=0, rollout_dp_rank=1)
    assert mine.prompts_by_dp == [[], [[3]], []] and mine.prompt_indices_by_dp == [[], [1], []]
    assert mine.max_cache_len == 9 and roll.prompts_by_dp[0] == [[1], [2]]          # the original is untouched
    score = narrow_for_rank(ScorePayload("ref", [[[1]], [[2]]], 7, 4), train_dp_rank=1, rollout_dp_rank=0)
    assert score.rows_by_dp == [[], [[2]]] and (score.role, score.pad_token_id, score.microbatch_size) == ("ref", 7, 4)
    a, b, whole = {"x": 1}, {"x": 2}, {"x": 3}
    train = narrow_for_rank(TrainPayload([[a, b], whole], 2), train_dp_rank=1, rollout_dp_rank=0)
    assert train.packs == [[None, b], whole] and train.gradient_accumulation_steps == 2
    critic = narrow_for_rank(TrainValuesPayload("critic", [[a, b]], None, 0.3, 0.7), train_dp_rank=0, rollout_dp_rank=0)
    assert critic.packs == [[a, None]] and critic.cliprange_value == 0.3
    cache = CachePayload(4, 128)
    assert narrow_for_rank(cache, train_dp_rank=0, rollout_dp_rank=0) is cache and narrow_for_rank(None, train_dp_rank=0, rollout_dp_rank=0) is None


def test_top_level_names_and_attribute_style_statistics():
    import copy
    import pickle

    import areno_b200
    from areno_b200.api import Trainer
    from areno_b200.engine.training import TrainStats

    assert areno_b200.Trainer is Trainer and areno_b200.ArenoEngine is ArenoEngine and areno_b200.EngineConfig is EngineConfig
    assert areno_b200.SamplingParams is SamplingParams and areno_b200.RolloutOutput is RolloutOutput
    assert areno_b200.TrainStats is TrainStats and areno_b200.ModelConfig is type(tiny_config())
    with pytest.raises(AttributeError):
        areno_b200.NoSuchName
    merged = merge_train_stats([{"loss": 1.0, "stepped": True, "metrics": {"kl": 0.5}}, {"loss": 2.0, "metrics": {"kl": 1.5}}])
    assert isinstance(merged, TrainStats) and merged.loss == merged["loss"] == 1.5 and merged.metrics == {"kl": 1.0}
    assert merged.stepped is True and merged == {"loss": 1.5, "stepped": True, "metrics": {"kl": 1.0}}
    with pytest.raises(AttributeError):
        merged.absent
    assert pickle.loads(pickle.dumps(merged)) == merged and copy.deepcopy(merged).loss == 1.5
    assert merge_train_stats([]) == {}


def test_the_engines_loss_function_is_the_default_for_packs_without_one(monkeypatch):
    seen = []

    def handler(op, payload, rank, dp_rank, tp_rank):
        seen.append([shards[dp_rank].get("_loss_fn") for shards in payload.packs])
        return [{"loss": 0.0, "metrics": {}} for _ in payload.packs]

    def engine_loss(pack, lp):
        return lp.sum()

    def pack_loss(pack, lp):
        return lp.mean()

    monkeypatch.setattr(engine_api, "make_cluster", lambda c, launcher, worker: ScriptedCluster(c, handler))
    cfg = EngineConfig(model=tiny_config(), train_loss_fn=engine_loss)
    eng = ArenoEngine(cfg)
    assert eng.loss_fn is engine_loss and eng.config.train_loss_fn is None and cfg.train_loss_fn is engine_loss
    eng.step([{"input_ids": torch.zeros(1, 2)}, {"input_ids": torch.zeros(1, 2), "_loss_fn": pack_loss}])
    assert seen[-1] == [engine_loss, pack_loss]
    explicit = ArenoEngine(cfg, loss_fn=pack_loss)
    assert explicit.loss_fn is pack_loss
    bare = ArenoEngine(EngineConfig(model=tiny_config()))
    bare.step([{"input_ids": torch.zeros(1, 2)}])
    assert seen[-1] == [None]                          # nothing stamped: the worker reports the missing loss


def test_model_configs_written_for_the_reference_construct():
    cfg = tiny_config(num_nextn_predict_layers=1, mtp_loss_scaling_factor=0.1, linear_backend="cublas", moe_backend="triton",
                      attn_backend="flash")
    assert cfg.num_nextn_predict_layers == 1 and cfg.attn_backend == "flash"


def test_the_engine_is_a_context_manager_that_closes_its_cluster(monkeypatch):
    closed = []
    eng, cluster = _engine(lambda *a: None, monkeypatch)
    cluster.close = lambda: closed.append(True)
    with eng as e:
        assert e is eng
    assert closed == [True]
    with pytest.raises(KeyError):
        with eng:
            raise KeyError("boom")
    assert closed == [True, True]
