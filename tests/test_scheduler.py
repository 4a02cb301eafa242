"""The scheduler's decisions: budget, portions, order, admission, what happens when pages run out."""

from __future__ import annotations

from liteinfer_b200.config.engine_config import EngineConfig
from liteinfer_b200.engine.scheduler import Scheduler, rows_to_shed
from liteinfer_b200.engine.sequence import Sequence, SequenceStatus, resolve_stop_status
from liteinfer_b200.sampling.params import SamplingParams


def _seq(name: str, prompt_len: int, **params) -> Sequence:
    return Sequence(name, "", list(range(prompt_len)), SamplingParams(**params))


def _run_step(sched: Scheduler):
    """Schedule one step and pretend it ran: counts advance, finished prompts sample one token."""
    out = sched.schedule()
    for seq in out.seqs:
        seq.num_computed_tokens += out.num_scheduled_tokens[seq.request_id]
        if seq.is_prompt_computed:
            seq.output_token_ids.append(0)
    return out


def test_a_prompt_larger_than_the_budget_is_cut_into_portions():
    sched = Scheduler(EngineConfig(model="m", max_num_seqs=2, max_num_batched_tokens=8))
    sched.add(_seq("a", 19))
    taken = []
    while not sched.running or not sched.running[0].is_prompt_computed:
        taken.append(_run_step(sched).num_scheduled_tokens["a"])
    assert taken == [8, 8, 3]
    assert _run_step(sched).num_scheduled_tokens == {"a": 1}       # then one token a step


def test_running_requests_come_first_and_newcomers_take_what_is_left():
    sched = Scheduler(EngineConfig(model="m", max_num_seqs=4, max_num_batched_tokens=10))
    sched.add(_seq("a", 3)); sched.add(_seq("b", 4))
    first = _run_step(sched)
    assert [s.request_id for s in first.seqs] == ["a", "b"] and first.num_scheduled_tokens == {"a": 3, "b": 4}
    sched.add(_seq("c", 20)); sched.add(_seq("d", 2))
    second = _run_step(sched)
    assert second.num_scheduled_tokens == {"a": 1, "b": 1, "c": 8}   # c takes all that is left; d waits behind it
    assert [s.request_id for s in sched.waiting] == ["d"]
    third = _run_step(sched)
    assert third.num_scheduled_tokens == {"a": 1, "b": 1, "c": 8}
    fourth = _run_step(sched)
    assert fourth.num_scheduled_tokens == {"a": 1, "b": 1, "c": 4, "d": 2}
    assert sum(fourth.num_scheduled_tokens.values()) <= 10


def test_no_step_exceeds_the_budget_and_every_prompt_token_is_computed_once():
    config = EngineConfig(model="m", max_num_seqs=3, max_num_batched_tokens=7)
    sched = Scheduler(config)
    seqs = [_seq(f"r{i}", n, max_tokens=4) for i, n in enumerate([5, 13, 1, 9, 22, 2])]
    for s in seqs:
        sched.add(s)
    computed = {s.request_id: 0 for s in seqs}
    for _ in range(200):
        if not sched.has_unfinished():
            break
        sched.remove_finished()
        out = sched.schedule()
        assert sum(out.num_scheduled_tokens.values()) <= 7 and len(sched.running) <= 3
        partial = [s for s in sched.running if not s.is_prompt_computed and s.num_computed_tokens > 0]
        assert len(partial) <= 1
        for seq in out.seqs:
            n = out.num_scheduled_tokens[seq.request_id]
            computed[seq.request_id] += n
            seq.num_computed_tokens += n
            if seq.is_prompt_computed:
                seq.output_token_ids.append(0)
                if seq.num_output_tokens >= 4:
                    seq.status = SequenceStatus.FINISHED_LENGTH
    assert not sched.has_unfinished() or all(s.is_finished for s in sched.running)
    for s in seqs:
        assert computed[s.request_id] == len(s.prompt_token_ids) + 3      # the last sampled token is never computed


def test_seats_limit_admission():
    sched = Scheduler(EngineConfig(model="m", max_num_seqs=2))
    for i in range(4):
        sched.add(_seq(f"r{i}", 2))
    assert len(_run_step(sched).seqs) == 2 and len(sched.waiting) == 2
    sched.running[0].status = SequenceStatus.FINISHED_STOPPED
    assert [s.request_id for s in sched.remove_finished()] == ["r0"]
    assert [s.request_id for s in _run_step(sched).seqs] == ["r1", "r2"]


class _Ledger:
    """A cache of `pages` pages of four tokens that keeps every key: what the scheduler asks of the cache manager."""

    def __init__(self, pages: int) -> None:
        self.pages = pages

    def can_hold(self, final_lengths, largest_step):
        return sum(-(-n // 4) for n in final_lengths) <= self.pages


def test_newcomers_wait_for_pages_instead_of_failing():
    ledger = _Ledger(4)                                     # a to its end (10 + 2 tokens) needs three pages
    sched = Scheduler(EngineConfig(model="m", max_num_seqs=4), ledger=ledger)
    sched.add(_seq("a", 10, max_tokens=2)); sched.add(_seq("b", 10, max_tokens=2))
    out = _run_step(sched)
    assert [s.request_id for s in out.seqs] == ["a"] and [s.request_id for s in sched.waiting] == ["b"]
    assert [s.request_id for s in _run_step(sched).seqs] == ["a"]     # b still waits; a decodes on
    ledger.pages = 6
    assert [s.request_id for s in _run_step(sched).seqs] == ["a", "b"]


def test_a_cache_that_holds_exactly_n_requests_seats_n_arriving_at_once():
    sched = Scheduler(EngineConfig(model="m", max_num_seqs=8), ledger=_Ledger(9))     # three pages a request
    for i in range(5):
        sched.add(_seq(f"r{i}", 10, max_tokens=2))
    assert [s.request_id for s in _run_step(sched).seqs] == ["r0", "r1", "r2"]
    assert len(sched.waiting) == 2


def test_a_request_that_can_never_fit_is_let_through_to_fail_alone():
    sched = Scheduler(EngineConfig(model="m", max_num_seqs=4), ledger=_Ledger(0))
    sched.add(_seq("huge", 50))
    assert [s.request_id for s in sched.schedule().seqs] == ["huge"]   # nothing runs: waiting would never end


def test_shedding_gives_up_the_least_invested_first():
    new, part, decoding = _seq("new", 5), _seq("part", 9), _seq("dec", 3)
    part.num_computed_tokens = 4
    decoding.num_computed_tokens = 3
    assert rows_to_shed([decoding, part, new]) == [new]
    assert rows_to_shed([decoding, part]) == [part]
    assert rows_to_shed([decoding]) == [decoding]


def test_stop_rules():
    seq = _seq("a", 3, max_tokens=5, min_tokens=2, stop_token_ids=[9])
    seq.output_token_ids = [7]
    assert resolve_stop_status(seq, 7, (7,), 100) is None                       # EOS before min_tokens
    seq.output_token_ids = [7, 7]
    assert resolve_stop_status(seq, 7, (7,), 100) == SequenceStatus.FINISHED_STOPPED
    assert resolve_stop_status(seq, 9, (), 100) == SequenceStatus.FINISHED_STOPPED
    assert resolve_stop_status(seq, 1, (), 100) is None
    assert resolve_stop_status(seq, 1, (), 5) == SequenceStatus.FINISHED_LENGTH  # max_model_len
    seq.output_token_ids = [1] * 5
    assert resolve_stop_status(seq, 1, (), 100) == SequenceStatus.FINISHED_LENGTH
    ignoring = _seq("b", 3, ignore_eos=True)
    ignoring.output_token_ids = [7]
    assert resolve_stop_status(ignoring, 7, (7,), 100) is None
    text = _seq("c", 3, stop=["END"])
    text.output_token_ids = [1]
    text.output_text = "the END"
    assert resolve_stop_status(text, 1, (), 100) == SequenceStatus.FINISHED_STOPPED


def test_portions_never_span_the_prompts_end():
    seq = _seq("a", 5)
    assert seq.next_tokens(5) == [0, 1, 2, 3, 4]
    seq.num_computed_tokens = 5
    seq.output_token_ids = [42]
    assert seq.next_tokens(1) == [42]
    seq.num_computed_tokens = 4
    try:
        seq.next_tokens(2)
    except ValueError:
        pass
    else:
        raise AssertionError("a portion spanning prompt and output was allowed")
