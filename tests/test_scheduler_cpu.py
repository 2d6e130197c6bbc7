"""The scheduler's decisions (C++ core alone, tokens handed in by the test), and the scheduler
above the step function with a CPU test double of the kernels against the plain implementation.
No GPU. What happens when pages run out is decided and tested here: the request that cannot
reserve ends with "capacity" and keeps what it generated; nobody waits, nobody is preempted."""
import pytest
import torch

import llmengine
import plain_llama as P
from cpu_ops import CpuOps
from llmengine.cache import host_module
from tiny import TINY_A, TINY_B, make_model_dir, random_ids

H = host_module()


def core(pages=64, page=4, slots=8, **kw):
    cm = H.CacheManager(page, [H.GroupSpec(pages, 0)], slots)
    return cm, H.SchedulerCore(cm, 256, 128, kw.pop("eos", set()), **kw)


def drain(s, token_of=lambda rid, k: 100 + k):
    """Runs the core with made-up tokens; returns the list of planned batches."""
    batches, count = [], {}
    while not s.idle:
        e = s.plan()
        if len(e):
            batches.append([(rid, e.tokens(i), e.want(i)) for i, rid in enumerate(e.ids())])
            toks = []
            for i, rid in enumerate(e.ids()):
                if e.want(i):
                    count[rid] = count.get(rid, 0) + 1
                    toks.append(token_of(rid, count[rid]))
            s.commit(toks)
    s.finalize()
    return batches


def test_knobs_and_enqueue_validation():
    cm, _ = core()
    with pytest.raises(ValueError, match="max_concurrent"):
        H.SchedulerCore(cm, 256, 128, set(), 0, 4)
    with pytest.raises(ValueError, match="max_prefill_tokens_per_step"):
        H.SchedulerCore(cm, 256, 128, set(), 4, 0)
    _, s = core()
    for bad, word in ((([], 1), "empty"), (([1], -1), "negative"), (([256], 1), "out of range"), (([-1], 1), "out of range"),
                      (([1] * 100, 29), "position limit")):
        with pytest.raises(ValueError, match=word):
            s.enqueue(*bad)
    with pytest.raises(ValueError, match="temperature"):
        s.enqueue([1], 1, -0.5)
    assert s.enqueue([1, 2], 1) == 0 and s.enqueue([3], 0) == 1
    s.budget = 7
    assert s.budget == 7
    with pytest.raises(ValueError):
        s.budget = 0


def test_budget_is_shared_first_come_first_served_and_decode_is_free():
    _, s = core(max_concurrent=8, max_prefill_tokens_per_step=8)
    a = s.enqueue(list(range(20)), 3)
    b = s.enqueue(list(range(50, 55)), 3)
    batches = drain(s)
    # step 0: a takes the whole budget; step 1: a again; step 2: a's last 4 and 4 of b; ...
    assert [(rid, len(t)) for rid, t, _ in batches[0]] == [(a, 8)]
    assert [(rid, len(t)) for rid, t, _ in batches[1]] == [(a, 8)]
    assert [(rid, len(t), w) for rid, t, w in batches[2]] == [(a, 4, [3]), (b, 4, [])]
    # step 3: b's last prompt token (wanted) beside a's first decoded token (not counted in the budget)
    assert [(rid, len(t), w) for rid, t, w in batches[3]] == [(b, 1, [0]), (a, 1, [0])]
    r = s.results
    assert [x.seq_id for x in r] == [0, 1] and all(x.finish_reason == "length" for x in r)
    assert list(r[0].token_ids) == list(range(20)) + [101, 102, 103] and r[0].prompt_len == 20


def test_admission_is_fifo_up_to_max_concurrent():
    cm, s = core(max_concurrent=2, max_prefill_tokens_per_step=64)
    for k in range(4):
        s.enqueue([k + 1] * 3, 2)
    e = s.plan()
    assert e.ids() == [0, 1] and s.num_waiting == 2 and s.last_admitted == [0, 1]
    s.commit([7, 7])
    drain(s)
    assert [r.seq_id for r in s.results] == [0, 1, 2, 3]
    assert cm.free_pages() == 64 and cm.free_slots == 8


def test_end_of_prompt_rules():
    _, s = core(eos={9})
    s.enqueue([1, 2, 3], 0)      # nothing sampled, "length"
    s.enqueue([1, 2, 3], 1)      # exactly one token
    s.enqueue([1, 2, 3], 5)      # EOS as first token: "stop", nothing appended
    s.enqueue([1, 2, 3], 5)      # EOS later
    toks = {1: [50], 2: [9], 3: [60, 61, 9, 62]}
    drain(s, lambda rid, k: toks[rid][k - 1])
    r = s.results
    assert [(list(x.token_ids), x.finish_reason) for x in r] == [
        ([1, 2, 3], "length"), ([1, 2, 3, 50], "length"), ([1, 2, 3], "stop"), ([1, 2, 3, 60, 61], "stop")]


def test_pages_run_out_the_request_that_cannot_reserve_ends_with_capacity():
    # The reference's case (tests/test_scheduler.py:285-307): 4 pages of 4; two requests of 4 + 12 tokens
    # need 4 pages each. Each holds two pages when the pool is empty; the first request is one token
    # ahead, asks for its third page first, cannot reserve and ends with "capacity"; its pages come
    # back at the next plan and the other finishes.
    cm, s = core(pages=4, page=4, max_concurrent=2, max_prefill_tokens_per_step=4)
    s.enqueue([1, 2, 3, 4], 12)
    s.enqueue([5, 6, 7, 8], 12)
    drain(s)
    r = s.results
    assert [x.finish_reason for x in r] == ["capacity", "length"]
    assert len(r[1].token_ids) == 16 and len(r[0].token_ids) == 9  # the loser keeps what it generated
    assert list(r[0].token_ids[:4]) == [1, 2, 3, 4]
    assert cm.free_pages() == 4 and cm.free_slots == 8  # everything came back
    cm.check()
    # With no page left at all, every request that needs one in that step ends (as in the reference,
    # where each failing row of the decode batch is marked dead, src/engine.cpp:581-589).
    cm, s = core(pages=4, page=4, max_concurrent=2, max_prefill_tokens_per_step=64)
    s.enqueue(list(range(8)), 8)
    s.enqueue(list(range(8)), 8)
    drain(s)
    assert [x.finish_reason for x in s.results] == ["capacity", "capacity"]
    assert all(len(x.token_ids) == 9 for x in s.results) and cm.free_pages() == 4
    # a prompt that can never fit ends with capacity at once and the next request still runs
    cm, s = core(pages=2, page=4, max_concurrent=1, max_prefill_tokens_per_step=64)
    s.enqueue(list(range(20)), 1)
    s.enqueue([1, 2], 1)
    drain(s)
    assert [x.finish_reason for x in s.results] == ["capacity", "length"]
    assert list(s.results[0].token_ids) == list(range(20))


def test_plan_commit_protocol():
    _, s = core()
    s.enqueue([1, 2], 2)
    s.plan()
    with pytest.raises(RuntimeError, match="not been committed"):
        s.plan()
    with pytest.raises(ValueError, match="expected 1 sampled"):
        s.commit([])
    s.commit([5])
    with pytest.raises(RuntimeError, match="no planned step"):
        s.commit([5])


# ------------------------------------------------------------------ with the step function (CPU double)
@pytest.fixture(scope="module", params=["a", "b"])
def engines(request, tmp_path_factory):
    cfg = {"a": TINY_A, "b": dict(TINY_B, eos_token_id=[3])}[request.param]
    d = str(tmp_path_factory.mktemp("model_" + request.param))
    make_model_dir(d, cfg, torch.float32)
    pc, pw = P.read_model(d)
    eng = llmengine.Engine(d, "fp32", device="cpu", ops=CpuOps(), block_size=4 if request.param == "a" else 16)
    return cfg, eng, pc, pw


def test_scheduler_equals_each_request_alone(engines):
    cfg, eng, pc, pw = engines
    lens = [5, 11, 17] if cfg is TINY_A else [1, 23, 40]
    prompts = [random_ids(n, cfg["vocab_size"], 40 + n) for n in lens]
    bm = llmengine.BlockManager(40, eng._default_block_size)
    sch = llmengine.ContinuousBatchScheduler(eng, bm, max_concurrent=3, max_prefill_tokens_per_step=7)
    for i, p in enumerate(prompts):
        sch.enqueue(p, [0, 1, 6][i])
    sch.run_until_idle()
    assert sch.idle and bm.free_blocks == 40
    for r, p, n in zip(sch.results, prompts, [0, 1, 6]):
        want, reason = P.generate(pc, pw, p, n)
        assert list(r.token_ids) == want and r.finish_reason == reason and r.prompt_len == len(p)
    eng.cm.check()


def test_temperature_sampling_does_not_depend_on_batching(engines):
    cfg, eng, pc, pw = engines
    prompts = [random_ids(n, cfg["vocab_size"], 90 + n) for n in (4, 9, 13)]
    alone = [eng.generate(p, 7, temperature=1.0, seed=100 + i) for i, p in enumerate(prompts)]
    sch = llmengine.ContinuousBatchScheduler(eng, llmengine.BlockManager(48, eng._default_block_size), 3, 5)
    for i, p in enumerate(prompts):
        sch.enqueue(p, 7, temperature=1.0, seed=100 + i)
    sch.run_until_idle()
    for r, (toks, reason), p, i in zip(sch.results, alone, prompts, range(3)):
        assert list(r.token_ids) == toks and r.finish_reason == reason
        assert (toks, reason) == P.generate(pc, pw, p, 7, temperature=1.0, seed=100 + i)
    assert alone[0][0] != eng.generate(prompts[0], 7, temperature=1.0, seed=999)[0]


def test_capacity_through_the_engine(engines):
    cfg, eng, pc, pw = engines
    bs = eng._default_block_size
    bm = llmengine.BlockManager(4, bs)
    sch = llmengine.ContinuousBatchScheduler(eng, bm, max_concurrent=2, max_prefill_tokens_per_step=256)
    p = random_ids(2 * bs, cfg["vocab_size"], 5)
    sch.enqueue(p, 2 * bs)
    sch.enqueue(p, 2 * bs)
    sch.run_until_idle()
    reasons = sorted(r.finish_reason for r in sch.results)
    assert "capacity" in reasons and bm.free_blocks == 4
    with pytest.raises(llmengine.CapacityError, match="KV pool exhausted"):
        eng.forward_logits_paged(random_ids(5 * bs, cfg["vocab_size"], 1), bm)
    assert bm.free_blocks == 4
    eng.cm.check()


def test_a_failed_step_ends_its_requests_with_error_and_the_others_go_on():
    cm, s = core(pages=16, page=4, max_concurrent=2, max_prefill_tokens_per_step=8)
    a = s.enqueue([1, 2, 3], 4)
    b = s.enqueue([4, 5], 4)
    c = s.enqueue([6], 2)  # waits: two may run at a time
    e = s.plan()
    assert e.ids() == [a, b]
    with pytest.raises(RuntimeError, match="no planned step"):
        core()[1].fail_step("error")
    s.fail_step("error")  # the device said that the step's results are void
    drain(s)
    r = {x.seq_id: x for x in s.results}
    assert r[a].finish_reason == "error" and list(r[a].token_ids) == [1, 2, 3]
    assert r[b].finish_reason == "error" and r[c].finish_reason == "length" and len(r[c].token_ids) == 3
    assert cm.free_pages() == 16 and cm.free_slots == 8
    cm.check()


def test_prompts_are_cut_at_multiples_of_what_the_model_asks_for():
    """A mixer that carries its state over only at the edges of chunks of M tokens asks for portions
    that end at multiples of M (parts.base.StateNeed.portion_multiple); the budget is then used up
    to the last such position, the end of a prompt is always a legal cut, and decoding is untouched."""
    cm, s = core(pages=64, page=4, max_concurrent=4, max_prefill_tokens_per_step=11, portion_multiple=4)
    assert s.portion_multiple == 4
    a = s.enqueue(list(range(23)), 2)
    b = s.enqueue(list(range(6)), 2)
    batches = drain(s)
    cuts = {a: [], b: []}
    for batch in batches:
        for rid, toks, _ in batch:
            if len(toks) > 1 or len(cuts[rid]) == 0 or sum(cuts[rid]) < (23 if rid == a else 6):
                cuts[rid].append(len(toks))
    # a: 8 (11 rounded down to a multiple of 4), 8, then its last 7; b gets what is left of each budget
    assert cuts[a][:3] == [8, 8, 7] and sum(cuts[a][:3]) == 23
    ends, pos = [], 0
    for n in cuts[b]:
        pos += n
        ends.append(pos)
        if pos == 6:
            break
    assert all(p % 4 == 0 or p == 6 for p in ends)
    assert all(x.finish_reason == "length" for x in s.results)
    with pytest.raises(ValueError, match="portion multiple"):
        core(max_prefill_tokens_per_step=3, portion_multiple=4)
    with pytest.raises(ValueError, match="portion multiple"):
        s.budget = 2


class _FailingOps(CpuOps):
    """The test double, reporting a kernel that gave up a wait at a chosen step (no kernel has to)."""

    ERROR_CODES = {22: "decoding attention: a tile never arrived"}

    def __init__(self):
        self.fail_at, self.checks = -1, 0

    def queue_error_check(self):
        self.checks += 1

    def take_step_error(self):
        return 22 if self.checks == self.fail_at else 0


def test_a_kernel_that_gave_up_raises_and_the_engine_stays_usable(tmp_path):
    d = str(tmp_path / "m")
    make_model_dir(d, TINY_A, torch.float32)
    pc, pw = P.read_model(d)
    ops = _FailingOps()
    eng = llmengine.Engine(d, "fp32", device="cpu", ops=ops, block_size=4, num_blocks=32)
    sch = llmengine.ContinuousBatchScheduler(eng, None, max_concurrent=2, max_prefill_tokens_per_step=64)
    p1, p2, p3 = (random_ids(n, 256, 70 + n) for n in (5, 7, 6))
    sch.enqueue(p1, 3)
    sch.enqueue(p2, 3)
    sch.enqueue(p3, 3)
    sch.step()
    ops.fail_at = ops.checks + 1  # the next step's kernels "give up"
    with pytest.raises(llmengine.KernelError, match="code 22.*a tile never arrived"):
        sch.step()
    sch.run_until_idle()
    r = sch.results
    assert [x.finish_reason for x in r] == ["error", "error", "length"]
    assert list(r[2].token_ids) == P.generate(pc, pw, p3, 3)[0]  # the request that was not in the failed step
    assert len(r[0].token_ids) == len(p1) + 1  # what was generated before the failure is kept
    eng.cm.check()
    assert eng.cm.free_pages(0) == 32 and eng.cm.free_slots == eng.cm.num_slots
    # the same through run_step: the error surfaces, fresh requests give their pages back
    ops.fail_at = ops.checks + 1
    with pytest.raises(llmengine.KernelError):
        eng.run_step([(5, p1, [0])])
    assert eng.cm.free_pages(0) == 32
