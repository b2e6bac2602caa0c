"""Scheduler through the C ABI with a mock executor (no GPU).

Re-expression of the reference's tests/test_scheduler.cpp:22-187: the mock returns one-hot
logits at request_id*100 + step, so arg-max sampling yields a known token sequence.
"""
import numpy as np

from mlcompiler_b200.host import CallbackExecutor, Scheduler

VOCAB = 1024


class MockExecutor(CallbackExecutor):
    def __init__(self):
        self.decode_calls, self.prefill_calls, self.released = {}, {}, set()
        self.last_decode_slots, self.max_slots = [], 0
        super().__init__()

    def _one_hot(self, tok):
        logits = np.full(VOCAB, -1e30, np.float32)
        logits[tok % VOCAB] = 1.0
        return logits

    def run_decode(self, slots):
        self.last_decode_slots = slots
        self.max_slots = max(self.max_slots, len(slots))
        out = []
        for rid, tok, pos in slots:
            self.decode_calls[rid] = self.decode_calls.get(rid, 0) + 1
            out.append((rid, True, self._one_hot(rid * 100 + self.decode_calls[rid])))
        return out

    def run_prefill(self, rid, tokens):
        self.prefill_calls[rid] = self.prefill_calls.get(rid, 0) + 1
        return self._one_hot(rid * 100)

    def release_request(self, rid):
        self.released.add(rid)


def test_empty_queue_is_idle():
    sched = Scheduler(MockExecutor())
    assert sched.empty() and sched.run_until_idle() == 0


def test_single_request_runs_to_completion():
    mock = MockExecutor()
    sched = Scheduler(mock, 8)
    rid = sched.add_request([1, 2, 3], max_new_tokens=5)
    assert rid == 1 and sched.queued_count() == 1
    emitted = []
    sched.set_token_callback(lambda r, t: emitted.append(t))
    sched.run_until_idle()
    assert sched.empty() and sched.completed_count() == 1
    assert len(emitted) == 5                      # first from prefill + 4 from decode
    assert emitted == [100, 101, 102, 103, 104]
    assert mock.prefill_calls[1] == 1 and mock.decode_calls[1] == 4
    assert 1 in mock.released
    drained = sched.drain_completed()
    assert len(drained) == 1 and drained[0]["state"] == Scheduler.COMPLETE
    assert len(drained[0]["generated_tokens"]) == 5


def test_multiple_requests_batched_together():
    mock = MockExecutor()
    sched = Scheduler(mock, 4)
    ids = [sched.add_request(p, max_new_tokens=3) for p in ([1, 2], [3, 4], [5, 6])]
    sched.run_until_idle()
    assert sched.completed_count() == 3
    for rid in ids:
        assert mock.prefill_calls[rid] == 1 and mock.decode_calls[rid] == 2
    assert len(mock.released) == 3
    st = sched.stats()
    assert st["total_requests_completed"] == 3 and st["total_tokens_generated"] == 9


def test_max_batch_size_bounds_active_set():
    mock = MockExecutor()
    sched = Scheduler(mock, 2)
    for p in ([1], [2], [3], [4]):
        sched.add_request(p, max_new_tokens=1)
    sched.tick()
    assert sched.active_count() <= 2
    sched.run_until_idle()
    assert sched.completed_count() == 4 and sched.empty()
    assert mock.max_slots <= 2


def test_eos_completes_early():
    mock = MockExecutor()
    sched = Scheduler(mock)
    sched.add_request([1], max_new_tokens=100, eos_token_id=100)   # first token = 1*100 + 0
    sched.run_until_idle()
    drained = sched.drain_completed()
    assert len(drained) == 1 and drained[0]["generated_tokens"] == [100]
    assert mock.decode_calls.get(1, 0) == 0


def test_iteration_level_admission_fills_vacancies():
    mock = MockExecutor()
    sched = Scheduler(mock, 2)
    sched.add_request([1], max_new_tokens=1)
    sched.add_request([2], max_new_tokens=1)
    sched.add_request([3], max_new_tokens=5)
    steps = sched.run_until_idle()
    assert steps > 0 and sched.completed_count() == 3 and sched.empty()


def test_decode_slots_carry_last_token_and_position():
    """slots = {id, last_token, position} (scheduler.cpp:96): position starts at the prompt
    length and advances by one per decode step."""
    mock = MockExecutor()
    sched = Scheduler(mock, 8)
    sched.add_request([7, 8, 9], max_new_tokens=3)
    sched.tick()   # admit + prefill (+ first decode in the same tick)
    assert mock.last_decode_slots == [(1, 100, 3)]
    sched.tick()
    assert mock.last_decode_slots == [(1, 101, 4)]


def test_failed_decode_marks_failed_and_releases():
    class Failing(MockExecutor):
        def run_decode(self, slots):
            return [(rid, False, None) for rid, _, _ in slots]
    mock = Failing()
    sched = Scheduler(mock, 4)
    sched.add_request([1], max_new_tokens=4)
    sched.run_until_idle()
    drained = sched.drain_completed()
    assert drained[0]["state"] == Scheduler.FAILED and 1 in mock.released


def test_prompt_less_request_goes_straight_to_decode():
    mock = MockExecutor()
    sched = Scheduler(mock, 4)
    sched.add_request([], max_new_tokens=2)
    sched.run_until_idle()
    assert mock.prefill_calls.get(1, 0) == 0 and mock.decode_calls[1] == 2
