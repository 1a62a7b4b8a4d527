"""Continuous-batching engine on the CPU runner: greedy output equals the whole-model path under chunked prefill,
prefix reuse and preemption; block accounting returns to a full pool."""
import pytest
import torch

from unillm_b200.config import GenerationConfig
from unillm_b200.engine.cpu_runner import CpuModelRunner
from unillm_b200.engine.llm_engine import LLMEngine
from unillm_b200.models import configs as C
from unillm_b200.models.families import LlamaModel, MixtralModel
from unillm_b200.sampling import SamplingParams

CASES = [
    (LlamaModel, C.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                               num_attention_heads=4, num_key_value_heads=2)),
    (MixtralModel, C.MixtralConfig(vocab_size=128, hidden_size=64, intermediate_size=64, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, num_experts=4, sliding_window=4096)),
]


def _prompts():
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 128, (13,), generator=g).tolist()
    return [shared + torch.randint(0, 128, (n,), generator=g).tolist() for n in (3, 9, 1, 6, 20, 2)]


@pytest.mark.parametrize("cls,cfg", CASES, ids=["llama", "mixtral"])
def test_engine_matches_model(cls, cfg):
    m = cls.new(cfg, init="random", seed=3)
    runner = CpuModelRunner(m, num_blocks=64, block_size=4, max_model_len=128)
    eng = LLMEngine(runner, num_blocks=64, block_size=4, max_num_seqs=4, max_num_batched_tokens=16, max_model_len=128)
    prompts = _prompts()
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    ref = [m.generate_ids(p, GenerationConfig.greedy(8, eos_token_id=-1)) for p in prompts]
    assert outs == ref
    assert eng.stats.cached_tokens > 0
    assert eng.pool.num_free() + eng.radix.stats()["cached_blocks"] == 64


def test_engine_preemption_keeps_outputs():
    cls, cfg = CASES[0]
    m = cls.new(cfg, init="random", seed=5)
    runner = CpuModelRunner(m, num_blocks=24, block_size=4, max_model_len=96)
    eng = LLMEngine(runner, num_blocks=24, block_size=4, max_num_seqs=4, max_num_batched_tokens=32, max_model_len=96,
                    enable_prefix_caching=False)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 128, (n,), generator=g).tolist() for n in (18, 17, 19, 16)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    ref = [m.generate_ids(p, GenerationConfig.greedy(12, eos_token_id=-1)) for p in prompts]
    assert outs == ref
    assert eng.stats.preemptions > 0
    assert eng.pool.num_free() == 24


def test_engine_abort_and_limits():
    cls, cfg = CASES[0]
    m = cls.new(cfg, init="random", seed=5)
    runner = CpuModelRunner(m, num_blocks=32, block_size=4, max_model_len=64)
    eng = LLMEngine(runner, num_blocks=32, block_size=4, max_num_seqs=4, max_num_batched_tokens=32, max_model_len=64)
    a = eng.add_request([1, 2, 3, 4, 5], SamplingParams(temperature=0.0, max_tokens=20))
    b = eng.add_request([1, 2, 3, 9], SamplingParams(temperature=0.0, max_tokens=5))
    eng.step()
    assert eng.abort(a) and not eng.abort(a)
    res = eng.run_to_completion()
    assert len(res[b]) == 5
    from unillm_b200.types import InvalidInput

    with pytest.raises(InvalidInput):
        eng.add_request(list(range(60)), SamplingParams(max_tokens=10))
    with pytest.raises(InvalidInput):
        eng.add_request([], SamplingParams())


def _run(async_scheduling, num_blocks, prompts, params, eos=None, prefix=True):
    cls, cfg = CASES[0]
    m = cls.new(cfg, init="random", seed=5)
    runner = CpuModelRunner(m, num_blocks=num_blocks, block_size=4, max_model_len=96)
    eng = LLMEngine(runner, num_blocks=num_blocks, block_size=4, max_num_seqs=4, max_num_batched_tokens=32,
                    max_model_len=96, enable_prefix_caching=prefix, eos_token_id=eos, async_scheduling=async_scheduling)
    ids = [eng.add_request(p, params) for p in prompts]
    streamed = {i: [] for i in ids}
    steps = 0
    while eng.has_unfinished():
        for o in eng.step():
            streamed[o.seq_id].append(o.token)
        steps += 1
        assert steps < 500
    outs = [eng.seqs[i].output_ids for i in ids]
    assert [streamed[i] for i in ids] == outs          # every token is reported exactly once, in order
    assert all(t >= 0 for o in outs for t in o)        # no placeholder survives
    return eng, outs


def test_async_scheduling_same_tokens():
    """One-step-ahead scheduling gives the tokens of the synchronous loop: plain decode, a stop token noticed one step
    late, and preemption while a step is in flight."""
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 128, (n,), generator=g).tolist() for n in (18, 17, 19, 16, 5, 30)]
    p = SamplingParams(temperature=0.0, max_tokens=12)
    e0, sync = _run(False, 64, prompts, p)
    e1, asyn = _run(True, 64, prompts, p)
    assert sync == asyn
    assert e1.pool.num_free() + e1.radix.stats()["cached_blocks"] == 64
    assert e1.stats.generated_tokens == e0.stats.generated_tokens
    # a stop token in the middle: take one that the greedy run produces
    eos = sync[0][4]
    _, s2 = _run(False, 64, prompts, p, eos=eos)
    e3, a2 = _run(True, 64, prompts, p, eos=eos)
    assert s2 == a2 and len(a2[0]) <= 5 and a2[0][-1] == eos
    assert e3.pool.num_free() + e3.radix.stats()["cached_blocks"] == 64
    # a small pool forces preemption
    e4, s3 = _run(False, 24, prompts[:4], p, prefix=False)
    e5, a3 = _run(True, 24, prompts[:4], p, prefix=False)
    assert s3 == a3 and e5.stats.preemptions > 0 and e5.pool.num_free() == 24


def test_async_scheduling_abort_and_snapshot():
    cls, cfg = CASES[0]
    m = cls.new(cfg, init="random", seed=5)
    runner = CpuModelRunner(m, num_blocks=32, block_size=4, max_model_len=64)
    eng = LLMEngine(runner, num_blocks=32, block_size=4, max_num_seqs=4, max_num_batched_tokens=32, max_model_len=64,
                    async_scheduling=True)
    a = eng.add_request([1, 2, 3, 4, 5], SamplingParams(temperature=0.0, max_tokens=20))
    b = eng.add_request([1, 2, 3, 9], SamplingParams(temperature=0.0, max_tokens=5))
    eng.step()
    eng.step()
    snap = eng.snapshot()
    assert all(t >= 0 for r in snap["requests"] for t in r["output"])
    assert eng.abort(a) and not eng.abort(a)
    res = eng.run_to_completion()
    assert len(res[b]) == 5 and all(t >= 0 for t in res[b])
    assert eng.pool.num_free() + eng.radix.stats()["cached_blocks"] == 32


def test_engine_allocates_from_finished_sequences_before_preempting():
    """With a small pool, the blocks cached for a finished request are evicted for a new one; the running request
    (whose published blocks are the oldest cache entries) is not preempted."""
    cls, cfg = CASES[0]
    m = cls.new(cfg, init="random", seed=5)
    runner = CpuModelRunner(m, num_blocks=16, block_size=4, max_model_len=64)
    eng = LLMEngine(runner, num_blocks=16, block_size=4, max_num_seqs=4, max_num_batched_tokens=64, max_model_len=64)
    g = torch.Generator().manual_seed(9)
    long_running = eng.add_request(torch.randint(0, 128, (17,), generator=g).tolist(),
                                   SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True))
    eng.step()                                     # prefill: 4 full blocks published while the sequence runs
    short = eng.add_request(torch.randint(0, 128, (21,), generator=g).tolist(),
                            SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    while eng.seqs[short].status != "finished":
        eng.step()
    third = eng.add_request(torch.randint(0, 128, (24,), generator=g).tolist(),
                            SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    while eng.seqs[third].status != "finished":
        eng.step()
    assert eng.stats.preemptions == 0
    assert eng.seqs[long_running].status == "running"


class _FlakyRunner:
    """Wraps a runner; ``fail_at`` lists the fetches (0-based) that report a device error instead of tokens."""

    def __init__(self, inner, fail_at):
        self.inner, self.fail_at, self.fetches, self.resets = inner, set(fail_at), 0, 0

    def launch(self, b):
        return self.inner.launch(b)

    def pending(self):
        return self.inner.pending()

    def fetch(self, handle=None):
        from unillm_b200.engine.runner import DeviceStepError

        k, self.fetches = self.fetches, self.fetches + 1
        if k in self.fail_at:
            raise DeviceStepError(2, 4000)
        return self.inner.fetch(handle)

    def reset_after_error(self):
        self.resets += 1


@pytest.mark.parametrize("async_sched", [False, True])
def test_engine_drops_a_step_whose_device_status_is_bad(async_sched):
    """A step whose error word reads 'flag wait timed out' hands no token to anybody and publishes nothing: the
    sequences are prefilled again from their history and the final outputs equal an undisturbed run."""
    cls, cfg = CASES[0]
    m = cls.new(cfg, init="random", seed=3)
    prompts = _prompts()
    ref = [m.generate_ids(p, GenerationConfig.greedy(8, eos_token_id=-1)) for p in prompts]
    runner = _FlakyRunner(CpuModelRunner(m, num_blocks=64, block_size=4, max_model_len=128), fail_at=[2, 5])
    eng = LLMEngine(runner, num_blocks=64, block_size=4, max_num_seqs=4, max_num_batched_tokens=16, max_model_len=128,
                    async_scheduling=async_sched)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    assert outs == ref
    assert eng.stats.device_errors == 2 and runner.resets == 2
    assert all(t >= 0 for o in outs for t in o)
    assert eng.pool.num_free() + eng.radix.stats()["cached_blocks"] == 64


def test_engine_raises_after_repeated_device_errors():
    from unillm_b200.engine.runner import DeviceStepError

    cls, cfg = CASES[0]
    m = cls.new(cfg, init="random", seed=3)
    runner = _FlakyRunner(CpuModelRunner(m, num_blocks=64, block_size=4, max_model_len=128), fail_at=range(100))
    eng = LLMEngine(runner, num_blocks=64, block_size=4, max_num_seqs=4, max_num_batched_tokens=16, max_model_len=128)
    eng.add_request([1, 2, 3], SamplingParams(temperature=0.0, max_tokens=4))
    with pytest.raises(DeviceStepError):
        for _ in range(10):
            eng.step()
