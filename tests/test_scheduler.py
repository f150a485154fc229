"""Scheduler / AsyncScheduler / EngineCore behaviour with a canned-token runner (host only).

Restates the behaviours pinned by the reference's tests/vllm/v1/test_scheduler.cpp,
test_async_scheduler.cpp, test_engine_core.cpp, test_engine_core_proc.cpp."""
import time

import pytest

from vllm_cpp_b200 import _engine as E

EOS = 7


def kv_cfg(num_blocks=100, block_size=4):
    spec = E.KVCacheSpec(kind=E.KVSpecKind.FULL_ATTENTION, block_size=block_size, num_kv_heads=1,
                         head_size=8)
    return E.KVCacheConfig(num_blocks, [E.KVCacheGroupSpec(["l0"], spec)])


def sched(budget=64, seqs=8, num_blocks=100, max_len=256, policy="fcfs", async_=False, caching=True):
    c = E.SchedulerConfig(max_num_batched_tokens=budget, max_num_seqs=seqs, max_model_len=max_len,
                          policy=policy, async_scheduling=async_, enable_prefix_caching=caching)
    return E.Scheduler(c, kv_cfg(num_blocks))


def req(rid, n=10, max_tokens=4, base=None, priority=0, arrival=0.0, **kw):
    if base is None:   # distinct prompts per request id unless a test wants a shared prefix
        base = 1000 * (1 + sum(ord(c) * (i + 1) for i, c in enumerate(rid)) % 97)
    sp = E.SamplingParams(max_tokens=max_tokens, **kw)
    return E.EngineCoreRequest(rid, [base + i for i in range(n)], sp, EOS, arrival, priority)


def mro(so, token=5, tokens=None):
    """Every request that finished its known tokens gets `token`."""
    o = E.ModelRunnerOutput()
    ids = list(so.num_scheduled_tokens.keys())
    o.req_ids = ids
    o.sampled_token_ids = [[(tokens or {}).get(i, token)] for i in ids]
    return o


def step(s, token=5, tokens=None, partial=()):
    so = s.schedule()
    m = mro(so, token, tokens)
    m.sampled_token_ids = [[] if r in partial else t for r, t in zip(m.req_ids, m.sampled_token_ids)]
    return so, s.update_from_output(so, m)


def test_fcfs_admits_all_under_budget():
    s = sched(budget=64)
    for i in range(3):
        s.add_request(req(f"r{i}", 10))
    so = s.schedule()
    assert so.num_scheduled_tokens == {"r0": 10, "r1": 10, "r2": 10}
    assert len(so.scheduled_new_reqs) == 3 and so.total_num_scheduled_tokens == 30
    assert s.num_running() == 3 and s.num_waiting() == 0


def test_budget_shared_and_chunked_prefill():
    s = sched(budget=16)
    s.add_request(req("a", 10))
    s.add_request(req("b", 10))
    so = s.schedule()
    assert so.num_scheduled_tokens == {"a": 10, "b": 6}   # b is chunked to fit
    s.update_from_output(so, mro_partial(so, partial={"b"}))
    so2 = s.schedule()
    # a decodes 1 token, b finishes its prompt; both appear as cached requests
    assert so2.num_scheduled_tokens == {"a": 1, "b": 4}
    assert so2.scheduled_new_reqs == [] and so2.scheduled_cached_reqs.req_ids == ["a", "b"]
    assert so2.scheduled_cached_reqs.new_token_ids[0] == [5]


def mro_partial(so, partial=(), token=5):
    m = mro(so, token)
    m.sampled_token_ids = [[] if r in partial else t for r, t in zip(m.req_ids, m.sampled_token_ids)]
    return m


def test_long_prompt_splits_over_steps_and_gets_no_token_while_prefilling():
    s = sched(budget=8)
    r = s.add_request(req("a", 20, max_tokens=2))
    so = s.schedule()
    assert so.num_scheduled_tokens == {"a": 8}
    outs = s.update_from_output(so, mro_partial(so, partial={"a"}))
    assert outs.outputs == [] and r.num_output_tokens == 0
    so = s.schedule()
    assert so.num_scheduled_tokens == {"a": 8}
    s.update_from_output(so, mro_partial(so, partial={"a"}))
    so = s.schedule()
    assert so.num_scheduled_tokens == {"a": 4}
    outs = s.update_from_output(so, mro(so))
    assert outs.outputs[0].new_token_ids == [5]


def test_late_prefill_joins_running_decode_and_max_num_seqs():
    s = sched(budget=32, seqs=2)
    s.add_request(req("a", 8))
    step(s)
    s.add_request(req("b", 8))
    s.add_request(req("c", 8))
    so = s.schedule()
    assert so.num_scheduled_tokens == {"a": 1, "b": 8}   # c waits: max_num_seqs = 2
    assert s.num_waiting() == 1


def test_stop_conditions():
    s = sched()
    a = s.add_request(req("a", 4, max_tokens=3))
    _, o = step(s)
    assert not o.outputs[0].finished()
    _, o = step(s)
    _, o = step(s)
    assert o.outputs[0].finished() and o.outputs[0].finish_reason == E.FinishReason.LENGTH
    assert a.status == E.RequestStatus.FINISHED_LENGTH_CAPPED and s.num_running() == 0
    # EOS
    s.add_request(req("b", 4, max_tokens=10))
    _, o = step(s, token=EOS)
    assert o.outputs[0].finish_reason == E.FinishReason.STOP and o.outputs[0].stop_reason is None
    # min_tokens blocks an early EOS
    s.add_request(req("c", 4, max_tokens=10, min_tokens=2))
    _, o = step(s, token=EOS)
    assert not o.outputs[0].finished()
    _, o = step(s, token=EOS)
    assert o.outputs[0].finished()
    # stop_token_ids set stop_reason
    s.add_request(req("d", 4, max_tokens=10, stop_token_ids=[42]))
    _, o = step(s, token=42)
    assert o.outputs[0].finish_reason == E.FinishReason.STOP and o.outputs[0].stop_reason.token == 42
    # ignore_eos keeps going
    s.add_request(req("e", 4, max_tokens=2, ignore_eos=True))
    so, o = step(s, token=EOS)
    assert not o.outputs[0].finished()
    # finished ids are reported to the worker on the next schedule, once
    assert so.finished_req_ids == {"d"}
    assert s.schedule().finished_req_ids == set()


def test_kv_exhaustion_preempts_tail_and_resumes_as_new():
    s = sched(budget=64, num_blocks=7, caching=False)  # 6 usable blocks of 4 tokens
    a = s.add_request(req("a", 11, max_tokens=20))
    b = s.add_request(req("b", 11, max_tokens=20, base=500))
    so, _ = step(s)            # 3 blocks each
    assert s.num_free_blocks() == 0
    so = s.schedule()          # a needs a 4th block at token 13 -> not yet; both decode token 12
    s.update_from_output(so, mro(so))
    so = s.schedule()          # now a needs block #4: b (tail) is preempted
    assert so.preempted_req_ids == ["b"]
    assert so.num_scheduled_tokens == {"a": 1}
    assert b.status == E.RequestStatus.PREEMPTED and b.num_computed_tokens == 0
    assert s.num_waiting() == 1 and b.num_preemptions == 1
    s.update_from_output(so, mro(so))
    s.finish_requests(["a"], E.RequestStatus.FINISHED_ABORTED)
    so = s.schedule()
    # resumed request re-enters as a new request carrying prompt + generated tokens
    assert [n.req_id for n in so.scheduled_new_reqs] == ["b"]
    assert len(so.scheduled_new_reqs[0].prompt_token_ids) == 11 + 2
    assert so.scheduled_new_reqs[0].num_prompt_tokens == 11
    assert so.num_scheduled_tokens == {"b": 13}


def test_priority_policy_ordering_and_victim():
    s = sched(budget=64, num_blocks=7, policy="priority", caching=False)
    s.add_request(req("low", 11, max_tokens=20, priority=5, arrival=1.0))
    s.add_request(req("high", 11, max_tokens=20, priority=0, arrival=2.0, base=300))
    so = s.schedule()
    assert list(so.num_scheduled_tokens.keys()) == ["high", "low"]   # priority, then arrival
    s.update_from_output(so, mro(so))
    so = s.schedule()
    s.update_from_output(so, mro(so))
    so = s.schedule()
    assert so.preempted_req_ids == ["low"]                            # victim = lowest priority
    assert "high" in so.num_scheduled_tokens
    # arrival tiebreak
    s2 = sched(policy="priority")
    s2.add_request(req("x", 4, priority=1, arrival=2.0))
    s2.add_request(req("y", 4, priority=1, arrival=1.0))
    assert list(s2.schedule().num_scheduled_tokens.keys()) == ["y", "x"]


def test_no_preemption_when_space_exists_and_abort_bookkeeping():
    s = sched()
    s.add_request(req("a", 8))
    s.add_request(req("b", 8))
    so, _ = step(s)
    assert so.preempted_req_ids == []
    s.finish_requests(["a", "nope"], E.RequestStatus.FINISHED_ABORTED)
    assert s.num_running() == 1 and s.get_request("a") is None
    so = s.schedule()
    assert "a" in so.finished_req_ids and "a" not in so.num_scheduled_tokens
    with pytest.raises(ValueError):
        s.add_request(req("b", 4))    # duplicate live id


def test_prefix_cache_hit_on_second_request():
    s = sched(budget=64)
    s.add_request(req("a", 16, max_tokens=1, base=100))
    step(s)
    r = s.add_request(req("b", 16, max_tokens=1, base=100))
    so = s.schedule()
    assert so.num_scheduled_tokens == {"b": 4} and r.num_cached_tokens == 12
    assert so.scheduled_new_reqs[0].num_computed_tokens == 12
    st = s.make_stats()
    assert st.prefix_cache_queries >= 16


def test_spec_decode_rollback():
    s = sched()
    r = s.add_request(req("a", 4, max_tokens=10))
    step(s)                                   # one token generated
    d = E.DraftTokenIds()
    d.req_ids, d.draft_token_ids = ["a"], [[11, 12, 13]]
    s.update_draft_token_ids(d)
    so = s.schedule()
    assert so.num_scheduled_tokens == {"a": 4}            # last token + 3 drafts
    assert so.scheduled_spec_decode_tokens == {"a": [11, 12, 13]}
    m = E.ModelRunnerOutput()
    m.req_ids, m.sampled_token_ids = ["a"], [[11, 99]]    # first draft accepted, then replaced
    before = r.num_computed_tokens
    o = s.update_from_output(so, m)
    assert o.outputs[0].new_token_ids == [11, 99]
    assert r.num_computed_tokens == before - 2            # two rejected drafts rolled back
    assert r.num_tokens == 4 + 1 + 2


# ------------------------------------------------------------------------- async scheduler
@pytest.mark.parametrize("max_tokens", [1, 2, 3, 5])
def test_async_stop_by_max_tokens(max_tokens):
    s = sched(async_=True)
    r = s.add_request(req("a", 6, max_tokens=max_tokens))
    pending = []
    produced = 0
    for _ in range(20):
        so = s.schedule()
        if so.total_num_scheduled_tokens:
            pending.append(so)
        if len(pending) == 2 or (pending and not so.total_num_scheduled_tokens):
            done = pending.pop(0)
            o = s.update_from_output(done, mro(done))
            produced += sum(len(x.new_token_ids) for x in o.outputs)
        if not s.has_unfinished_requests() and not pending:
            break
    assert produced == max_tokens and r.num_output_tokens == max_tokens
    assert r.num_output_placeholders == 0


def test_async_schedules_ahead_with_placeholder():
    s = sched(async_=True)
    r = s.add_request(req("a", 6, max_tokens=8))
    so1 = s.schedule()
    assert r.num_output_placeholders == 1
    so2 = s.schedule()                       # next decode scheduled before the token is known
    assert so2.num_scheduled_tokens == {"a": 1}
    assert so2.scheduled_cached_reqs.new_token_ids == [[]]   # token still in flight
    s.update_from_output(so1, mro(so1))
    assert r.num_output_tokens == 1 and r.num_output_placeholders == 1


# ----------------------------------------------------------------------------- engine core
class CannedRunner(E.ModelRunnerBase):
    def __init__(self, token=5, fail_at=None, delay=0.0):
        super().__init__()
        self.delay = delay
        self.calls = []
        self.token = token
        self.fail_at = fail_at
        self.n = 0

    def execute_model(self, so):
        if so.total_num_scheduled_tokens == 0:
            return
        self.n += 1
        if self.delay:
            time.sleep(self.delay)
        if self.fail_at is not None and self.n >= self.fail_at:
            raise RuntimeError("injected runner failure")
        self.calls.append("execute")
        self._ids = list(so.num_scheduled_tokens.keys())
        self._known = {}

    def sample_tokens(self, grammar):
        self.calls.append("sample" if grammar is None else "sample+grammar")
        o = E.ModelRunnerOutput()
        o.req_ids = self._ids
        o.sampled_token_ids = [[self.token] for _ in self._ids]
        return o


def core(runner, **kw):
    c = E.SchedulerConfig(max_num_batched_tokens=64, max_num_seqs=8, max_model_len=256,
                          async_scheduling=kw.get("async_", False))
    return E.EngineCore(c, kv_cfg(), runner, kw.get("depth", 1))


def test_engine_core_step_order_and_empty_step():
    r = CannedRunner()
    c = core(r)
    outs, executed = c.step()
    assert not executed and r.calls == []
    c.add_request(req("a", 4, max_tokens=2))
    outs, executed = c.step()
    assert executed and r.calls == ["execute", "sample"]
    assert outs.outputs[0].new_token_ids == [5]
    c.abort_requests(["a"])
    outs, executed = c.step()
    assert not executed
    with pytest.raises(ValueError):
        c.add_request(req("bad", 4, temperature=-1.0))


def test_batch_queue_finishes_every_request_once():
    r = CannedRunner()
    c = core(r, async_=True, depth=2)
    for i in range(3):
        c.add_request(req(f"r{i}", 4 + i, max_tokens=3))
    finished, tokens = [], {}
    for _ in range(50):
        outs, _ = c.step_with_batch_queue()
        for o in outs.outputs:
            tokens[o.request_id] = tokens.get(o.request_id, 0) + len(o.new_token_ids)
            if o.finished():
                finished.append(o.request_id)
        if not c.has_work():
            break
    assert sorted(finished) == ["r0", "r1", "r2"]
    assert tokens == {"r0": 3, "r1": 3, "r2": 3}


def _drain(c, want, timeout=10.0):
    got, t0 = {}, time.time()
    while len([k for k, v in got.items() if v]) < want and time.time() - t0 < timeout:
        o = c.get_output(0.5)
        if o is None:
            continue
        for x in o.outputs:
            got[x.request_id] = got.get(x.request_id, False) or x.finished()
    return got


def test_busy_loop_cycle_abort_and_shutdown():
    c = core(CannedRunner(delay=0.005))
    c.start_busy_loop()
    c.add_request_async(req("a", 4, max_tokens=3))
    c.add_request_async(req("b", 4, max_tokens=100))
    got = _drain(c, 1)
    assert got.get("a")
    c.abort_requests_async(["b"])
    c.abort_requests_async(["a"])        # abort after finish: no-op
    time.sleep(0.2)
    c.add_request_async(req("c", 4, max_tokens=1000))
    time.sleep(0.1)
    c.shutdown(True)                      # abort mode: c ends with a terminal abort output
    saw_abort = False
    while True:
        o = c.get_output(0.2)
        if o is None:
            break
        for x in o.outputs:
            if x.request_id == "c" and x.finished() and x.finish_reason == E.FinishReason.ABORT:
                saw_abort = True
    assert saw_abort


def test_idle_shutdown_wakes_up():
    c = core(CannedRunner())
    c.start_busy_loop()
    t0 = time.time()
    c.shutdown(True)
    assert time.time() - t0 < 2.0


def test_runner_failure_marks_engine_dead():
    c = core(CannedRunner(fail_at=2))
    c.start_busy_loop()
    c.add_request_async(req("a", 4, max_tokens=10))
    with pytest.raises(E.EngineDeadError):
        for _ in range(50):
            c.get_output(1.0)
    assert c.engine_dead()
    with pytest.raises(E.EngineDeadError):
        c.add_request_async(req("b", 4))
    c.shutdown(True)


class AsyncLoadConnector(E.KVConnectorHook):
    """A connector that answers "N tokens are available remotely and will arrive asynchronously"
    and asks for the blocks of finished requests to be kept while it sends them."""

    def __init__(self, external_tokens, delay_free=False):
        super().__init__()
        self.external, self.delay = external_tokens, delay_free
        self.alloc = []

    def get_num_new_matched_tokens(self, rid, token_ids, num_computed):
        return (max(0, self.external - num_computed), True)

    def update_state_after_alloc(self, rid, token_ids, block_ids, num_external):
        self.alloc.append((rid, [list(b) for b in block_ids], num_external))

    def request_finished(self, rid, token_ids, block_ids, num_computed):
        return self.delay


def test_async_remote_kv_load_is_promoted_when_the_runner_reports_it():
    """A request whose prefix loads asynchronously holds its blocks and computes nothing until
    the runner names it in finished_recving; then only the rest of the prompt is scheduled."""
    conn = AsyncLoadConnector(external_tokens=8)
    c = E.SchedulerConfig(max_num_batched_tokens=64, max_num_seqs=8, max_model_len=256)
    s = E.Scheduler(c, kv_cfg(100, block_size=4), conn)
    s.add_request(req("a", 10, max_tokens=2))
    free0 = s.num_free_blocks()
    so = s.schedule()
    assert so.total_num_scheduled_tokens == 0 and s.num_waiting() == 1 and s.num_running() == 0
    assert conn.alloc and conn.alloc[0][2] == 8 and s.num_free_blocks() == free0 - 2
    s.update_from_output(so, E.ModelRunnerOutput())
    # not reported yet: still parked, every step
    so = s.schedule()
    assert so.total_num_scheduled_tokens == 0 and s.num_waiting() == 1
    done = E.ModelRunnerOutput()
    done.finished_recving = {"a"}
    s.update_from_output(so, done)
    so = s.schedule()
    assert so.num_scheduled_tokens == {"a": 2}          # 10 prompt tokens - 8 loaded
    assert s.num_running() == 1 and s.num_waiting() == 0
    s.update_from_output(so, mro(so))
    so, outs = step(s)
    assert outs.outputs[0].finish_reason is not None and s.num_free_blocks() == free0


def test_delayed_free_releases_blocks_on_finished_sending():
    conn = AsyncLoadConnector(external_tokens=0, delay_free=True)
    conn.get_num_new_matched_tokens = lambda rid, toks, n: (0, False)
    c = E.SchedulerConfig(max_num_batched_tokens=64, max_num_seqs=8, max_model_len=256)
    s = E.Scheduler(c, kv_cfg(100, block_size=4), conn)
    free0 = s.num_free_blocks()
    s.add_request(req("a", 10, max_tokens=1))
    so, outs = step(s)
    assert outs.outputs[0].finish_reason is not None
    assert s.num_delayed_free() == 1 and s.num_free_blocks() < free0    # the connector still sends
    so = s.schedule()
    sent = E.ModelRunnerOutput()
    sent.finished_sending = {"a"}
    s.update_from_output(so, sent)
    assert s.num_delayed_free() == 0 and s.num_free_blocks() == free0
