"""The scheduler's decisions, on the host (no GPU): portions under the budget, first-in
first-out admission, what happens when pages run out (src/engine.cpp:304-377)."""
import pytest

from bitwise_b200.cache import CacheManager, GroupSpec
from bitwise_b200.engine.scheduler import Scheduler, Sequence
from bitwise_b200.sampling import SamplingParams


def make(pages, budget, max_seqs, page=16):
    m = CacheManager([GroupSpec(None, (0,))], [pages], page, max_seqs)
    return m, Scheduler(m, budget, max_seqs)


def seq(i, n, new=8):
    return Sequence(i, list(range(n)), n, SamplingParams(max_new_tokens=new))


def run(plan):
    """Pretend the step ran: everything planned is computed; finished prompts get a token."""
    for p in plan:
        p.seq.computed += p.n
        if p.seq.computed == len(p.seq.tokens):
            p.seq.tokens.append(1)


def shape(plan):
    return [(p.seq.id, p.n) for p in plan]


def test_prompts_are_cut_into_portions_under_the_budget():
    m, s = make(64, 24, 8)
    a, b = seq(0, 40), seq(1, 10)
    s.add(a), s.add(b)
    assert shape(p := s.plan()) == [(0, 24)]          # the head takes the whole budget; b waits
    run(p)
    assert shape(p := s.plan()) == [(0, 16), (1, 8)]   # running first, then the newcomer gets the rest
    run(p)
    assert shape(p := s.plan()) == [(0, 1), (1, 2)]    # a decodes, b finishes its prompt
    run(p)
    assert shape(s.plan()) == [(0, 1), (1, 1)]


def test_admission_is_first_in_first_out_and_stops_at_the_head():
    m, s = make(4, 128, 8)                             # 64 tokens of cache
    big, small = seq(0, 70), seq(1, 5)                 # the head can not get its pages
    s.add(big), s.add(small)
    assert s.plan() == [] and not m.has(0) and m.available() == 4  # gave back what it took; nobody behind it is tried
    assert [q.id for q in s.waiting] == [0, 1]


def test_max_num_seqs_limits_admission():
    m, s = make(64, 64, 2)
    for i in range(3):
        s.add(seq(i, 4))
    assert shape(s.plan()) == [(0, 4), (1, 4)] and len(s.waiting) == 1


def test_youngest_unscheduled_running_request_is_preempted():
    m, s = make(6, 128, 8)                             # 96 tokens
    a, b, c = seq(0, 30), seq(1, 30), seq(2, 30)
    for q in (a, b, c):
        s.add(q)
    run(s.plan())                                       # all admitted: 2 pages each, pool empty
    assert m.available() == 0
    a.tokens += [1] * 2                                 # a now needs a third page (33 tokens)
    b.tokens += [1] * 2
    plan = s.plan()
    # a asks first: victim is the youngest running one not yet scheduled and not a -> c.
    # b then finds a free page (c had two). c went back to the queue and was re-admitted with
    # what is left, or waits.
    assert s.preempted_log == [2]
    assert (0, 3) in shape(plan) and (1, 3) in shape(plan)
    assert c.computed == 0 or c.running
    m.check_consistency()


def test_preempted_request_returns_in_id_order_and_is_recomputed():
    m, s = make(4, 64, 8)
    a, b = seq(0, 30), seq(1, 30)
    s.add(a), s.add(b)
    run(s.plan())
    newcomer = seq(2, 5)
    s.add(newcomer)
    a.tokens += [1] * 3                                 # a: 34 tokens -> third page; pool is empty
    plan = s.plan()
    assert s.preempted_log == [1] and [q.id for q in s.waiting][0] == 1  # ahead of the newer arrival
    assert b.computed == 0 and not b.running and not m.has(1)
    assert shape(plan)[0] == (0, 4)
    run(plan)
    # later b runs again from position 0 over prompt + what it had generated
    a_done = s.finish(a)
    plan = s.plan()
    assert shape(plan)[0] == (1, len(b.tokens))


def test_a_request_alone_preempts_itself_when_nothing_else_can_go():
    m, s = make(2, 64, 8)
    a = seq(0, 30)
    s.add(a)
    run(s.plan())
    a.tokens += [1] * 5                                 # 36 tokens: needs a third page, there is none
    plan = s.plan()
    assert s.preempted_log == [0]
    # it re-enters the queue, and at admission the head can not get 3 pages either: nothing runs
    assert plan == [] and m.available() == 2


def test_finish_gives_everything_back():
    m, s = make(8, 64, 4)
    a, b = seq(0, 20), seq(1, 3)
    s.add(a), s.add(b)
    run(s.plan())
    s.finish(a)
    assert [q.id for q in s.running] == [1] and m.available() == 7
    s.finish(b)
    assert s.idle() and m.all_free()
