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


class CursorMock(MockExecutor):
    """Remembers how far every request's prefill has come, like the executor does (known_position)."""

    def __init__(self):
        self.fed, self.chunks, self.events = {}, {}, []
        super().__init__()

    def run_prefill(self, rid, tokens):
        self.chunks.setdefault(rid, []).append(list(tokens))
        self.fed[rid] = self.fed.get(rid, 0) + len(tokens)
        self.events.append(("prefill", rid, len(tokens)))
        return super().run_prefill(rid, tokens)

    def run_decode(self, slots):
        self.events.append(("decode", tuple(s[0] for s in slots)))
        return super().run_decode(slots)


def test_chunked_admission_feeds_a_prompt_in_pieces_and_keeps_decoding():
    """A long prompt arrives while another request is decoding: with chunked admission the prompt goes
    in 4 tokens per tick and the other request gets a decode step on every one of those ticks; the
    generated tokens are the same as without chunking."""
    results = {}
    for chunk in (0, 4):
        mock = CursorMock()
        sched = Scheduler(mock, 8)
        sched.set_prefill_chunk_tokens(chunk)
        a = sched.add_request([5], max_new_tokens=12)
        sched.tick()                                  # request a: prefilled, first decode done
        b = sched.add_request(list(range(100, 110)), max_new_tokens=3)     # 10 prompt tokens
        emitted = {}
        sched.set_token_callback(lambda r, t: emitted.setdefault(r, []).append(t))
        sched.run_until_idle()
        done = {d["id"]: d["generated_tokens"] for d in sched.drain_completed()}
        results[chunk] = done
        if chunk:
            assert mock.chunks[b] == [[100, 101, 102, 103], [104, 105, 106, 107], [108, 109]]
            assert mock.fed[b] == 10 and sched.prefill_calls() == 1 + 3
            # between the first and the last chunk of b, request a decoded on every tick
            idx = [i for i, e in enumerate(mock.events) if e[0] == "prefill" and e[1] == b]
            between = mock.events[idx[0]:idx[-1]]
            assert sum(1 for e in between if e[0] == "decode" and a in e[1]) == 2
            # b joins the decode pass only after its last chunk
            first_b_decode = next(i for i, e in enumerate(mock.events) if e[0] == "decode" and b in e[1])
            assert first_b_decode > idx[-1]
        else:
            assert mock.chunks[b] == [list(range(100, 110))] and sched.prefill_calls() == 2
    assert results[0] == results[4]
    assert len(results[4][1]) == 12 and len(results[4][2]) == 3


def test_chunk_larger_than_the_prompt_is_one_call():
    mock = CursorMock()
    sched = Scheduler(mock, 2)
    sched.set_prefill_chunk_tokens(64)
    rid = sched.add_request([1, 2, 3], max_new_tokens=2)
    sched.run_until_idle()
    assert mock.chunks[rid] == [[1, 2, 3]] and sched.prefill_calls() == 1
    assert sched.completed_count() == 1


def test_failed_chunk_fails_the_request_and_releases_it():
    class FailSecond(CursorMock):
        def run_prefill(self, rid, tokens):
            out = super().run_prefill(rid, tokens)
            return np.zeros(0, np.float32) if len(self.chunks[rid]) == 2 else out    # empty logits = failure

    mock = FailSecond()
    sched = Scheduler(mock, 2)
    sched.set_prefill_chunk_tokens(2)
    rid = sched.add_request([1, 2, 3, 4, 5], max_new_tokens=4)
    sched.run_until_idle()
    d = sched.drain_completed()
    assert len(d) == 1 and d[0]["state"] == Scheduler.FAILED and d[0]["generated_tokens"] == []
    assert rid in mock.released
