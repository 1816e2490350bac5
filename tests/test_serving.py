"""Host-side scheduler: resources are never shared between live sequences, every request gets
exactly its tokens, and the outputs do not depend on how steps were packed (checked with a fake
executor whose next token is a function of the sequence's own history)."""
import numpy as np
import pytest

from logismos_b200.serving import Request, Scheduler, serve, shard_requests, synthetic_load


class FakeExecutor:
    """Keeps each sequence's history by state slot and checks the scheduler's bookkeeping."""

    def __init__(self):
        self.hist = {}
        self.block_owner = {}

    def __call__(self, plan):
        out, off = [], 0
        assert len(set(plan.slots.tolist())) == len(plan.rids)
        for i, rid in enumerate(plan.rids):
            n, c, slot = int(plan.new[i]), int(plan.cached[i]), int(plan.slots[i])
            toks = plan.ids[off:off + n].tolist(); off += n
            if c == 0:
                self.hist[slot] = (rid, [])
            owner, h = self.hist[slot]
            assert owner == rid and len(h) == c, "slot reused while its sequence is live, or wrong cached length"
            h.extend(toks)
            row = plan.tables[i]
            assert (row[: -(-len(h) // 16)] >= 0).all()
            for b in row[row >= 0].tolist():
                assert self.block_owner.setdefault(b, rid) == rid, "KV block shared by two live sequences"
            out.append((sum(h) * 2654435761 + len(h)) % 1000)
        assert off == plan.ids.size
        return np.asarray(out, np.uint32)


def alone(req):
    h, out = req.prompt.tolist(), []
    for _ in range(req.max_new):
        t = (sum(h) * 2654435761 + len(h)) % 1000
        out.append(t); h.append(t)
    return out


class Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        self.t += 0.01
        return self.t


@pytest.mark.parametrize("budget,seqs", [(4096, 64), (600, 5), (513, 2)])
def test_outputs_do_not_depend_on_packing(budget, seqs):
    reqs = synthetic_load(40, 3, 1000, prompt_median=60, prompt_sigma=0.8, prompt_cap=512, out_lo=1, out_hi=24, rate_per_s=50.0)
    sched = Scheduler(n_pool_blocks=200, max_blocks_per_seq=40, n_state_slots=seqs, max_step_tokens=budget, max_step_seqs=seqs)
    ex = FakeExecutor()

    def step(plan):
        toks = ex(plan)
        return toks

    def on_step(plan):  # blocks of finished sequences go back to the pool: forget their owner
        live = {b for r in sched.tables.values() for b in r[r >= 0].tolist()}
        for b in list(ex.block_owner):
            if b not in live:
                del ex.block_owner[b]

    steps = serve(step, sched, reqs, Clock(), on_step=on_step)
    assert steps > 0 and sched.idle() and len(sched.done) == 40
    assert len(sched.free_blocks) == 200 and len(set(sched.free_blocks)) == 200 and len(sched.free_slots) == seqs
    assert sched.generated == sum(r.max_new for r in reqs) and sched.prefilled == sum(len(r.prompt) for r in reqs)
    for r in reqs:
        assert r.output == alone(r)
        assert r.first_token_at >= r.arrival and r.finished_at >= r.first_token_at


@pytest.mark.parametrize("budget,step_tokens,seqs", [(64, 96, 8), (17, 48, 3), (150, 200, 16)])
def test_chunked_prefill_feeds_prompts_in_pieces_with_the_same_outputs(budget, step_tokens, seqs):
    """Prompts longer than a step are fed in chunks against their cached prefix; a chunk that does not
    end its prompt produces no token; outputs equal those of each request run alone."""
    reqs = synthetic_load(30, 5, 1000, prompt_median=90, prompt_sigma=0.9, prompt_cap=512, out_lo=1, out_hi=12, rate_per_s=80.0)
    assert max(len(r.prompt) for r in reqs) > step_tokens  # some prompt cannot fit one step
    sched = Scheduler(n_pool_blocks=400, max_blocks_per_seq=40, n_state_slots=seqs, max_step_tokens=step_tokens, max_step_seqs=seqs,
                      prefill_token_budget=budget, chunked_prefill=True)
    ex = FakeExecutor()
    seen = []

    def step(plan):
        assert int(plan.new.sum()) <= step_tokens and plan.n_prefill_tokens <= budget
        seen.append(plan)
        return ex(plan)

    def on_step(plan):
        live = {b for r in sched.tables.values() for b in r[r >= 0].tolist()}
        for b in list(ex.block_owner):
            if b not in live:
                del ex.block_owner[b]

    serve(step, sched, reqs, Clock(), on_step=on_step)
    assert sched.idle() and len(sched.done) == 30 and not sched.prefilling
    assert len(sched.free_blocks) == 400 and len(sched.free_slots) == seqs
    assert sched.generated == sum(r.max_new for r in reqs) and sched.prefilled == sum(len(r.prompt) for r in reqs)
    assert any((p.cached[p.n_decode:] > 0).any() for p in seen), "no chunk ever continued a cached prefix"
    assert any(not p.emits.all() for p in seen)
    for r in reqs:
        assert r.output == alone(r)


def test_requests_that_can_never_run_are_refused_and_load_is_seeded():
    sched = Scheduler(n_pool_blocks=8, max_blocks_per_seq=4, n_state_slots=2, max_step_tokens=32, max_step_seqs=2)
    with pytest.raises(ValueError):
        sched.add(Request(0, np.ones(60, np.uint32), 10))      # more blocks than a table row
    with pytest.raises(ValueError):
        sched.add(Request(1, np.ones(40, np.uint32), 1))       # prompt larger than a step
    a = synthetic_load(64, 9, 151936, rate_per_s=100.0)
    b = synthetic_load(64, 9, 151936, rate_per_s=100.0)
    assert all(np.array_equal(x.prompt, y.prompt) and x.max_new == y.max_new and x.arrival == y.arrival for x, y in zip(a, b))
    lens = np.array([len(r.prompt) for r in synthetic_load(4000, 1, 1000)])
    assert lens.max() <= 16384 and 900 < np.median(lens) < 1150
    assert all(64 <= r.max_new <= 1024 for r in a)
    parts = [shard_requests(a, 4, r) for r in range(4)]
    assert sorted(x.rid for p in parts for x in p) == list(range(64)) and all(len(p) == 16 for p in parts)


def test_stalled_pool_is_reported():
    sched = Scheduler(n_pool_blocks=2, max_blocks_per_seq=4, n_state_slots=2, max_step_tokens=64, max_step_seqs=2)
    with pytest.raises(RuntimeError):
        serve(lambda p: np.zeros(len(p.rids), np.uint32), sched, [Request(0, np.ones(40, np.uint32), 8)], Clock())


def test_decode_chunk_choice_follows_the_cta_count():
    """logismos_pick_decode_chunk: the largest of 512 / 1024 / 2048 tokens that leaves chunks x kv heads
    >= 32768 / head_dim CTAs; 512 when neither does (host-side arithmetic only)."""
    import ctypes as C
    from logismos_b200._lib import lib

    def pick(ctx, n_kv, d):
        a = np.ascontiguousarray(ctx, dtype=np.int32)
        return lib.logismos_pick_decode_chunk(a.ctypes.data_as(C.c_void_p), a.size, n_kv, d)

    assert pick([1500] * 256, 2, 256) == 2048   # 256 chunks x 2 heads
    assert pick([1500] * 32, 2, 256) == 1024    # 2048 would leave 64 CTAs, 1024 leaves 128
    assert pick([100] * 4, 2, 256) == 512
    assert pick([4000] * 64, 2, 128) == 2048    # 128 chunks x 2 = 256 = 32768 / 128
    assert pick([4000] * 63, 2, 128) == 1024
    assert pick([], 2, 128) == 512 and pick([5, -3, 0], 2, 128) == 512
