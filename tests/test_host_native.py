"""The native host runtime (include/iian_b200, iian_b200/csrc/host) against the same algorithms in plain Python
(tests/plain_block_pool.py, plain_cache_manager.py, plain_scheduler.py), operation by operation under random
sequences: same pages in the same order, same tables, same hashes, same scheduling decisions."""
import random

import pytest

import plain_block_pool as ppool
import plain_cache_manager as pcache
import plain_scheduler as psched
from iian_b200.cache.block_pool import BlockPool, PoolError, hash_block
from iian_b200.cache.manager import CacheManager, PageGroup
from iian_b200.config.engine import SchedulerConfig
from iian_b200.engine.request import Request
from iian_b200.engine.scheduler import Scheduler
from iian_b200.sampling.params import SamplingParams


def test_hash_is_the_same_function():
    rng = random.Random(0)
    for _ in range(200):
        toks = [rng.randrange(0, 200000) for _ in range(rng.randrange(1, 40))]
        parent, salt = rng.getrandbits(64), rng.getrandbits(64) if rng.random() < 0.3 else 0
        assert hash_block(parent, toks, salt) == ppool.hash_block(parent, toks, salt)
    assert hash_block(0, [1, 2, 3]) != 0


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("caching", [True, False])
def test_block_pool_matches_the_plain_pool(seed, caching):
    rng = random.Random(seed)
    bs, nb = 4, 12
    a, b = BlockPool(nb, bs, caching), ppool.BlockPool(nb, bs, caching)
    held = []
    pages_of_tokens = [[rng.randrange(9) for _ in range(bs)] for _ in range(5)]
    for _ in range(600):
        op = rng.random()
        if op < 0.35:
            n = rng.randrange(0, 5)
            if n > a.num_free:
                with pytest.raises(PoolError):
                    a.get_new_blocks(n)
                with pytest.raises(ppool.PoolError):
                    b.get_new_blocks(n)
            else:
                got = a.get_new_blocks(n)
                assert got == b.get_new_blocks(n)
                held += got
        elif op < 0.6 and held:
            k = rng.randrange(1, min(4, len(held)) + 1)
            pick = [held.pop(rng.randrange(len(held))) for _ in range(k)]
            a.free_blocks(pick)
            b.free_blocks(pick)
        elif op < 0.8 and held:
            p = rng.choice(held)
            toks = rng.choice(pages_of_tokens)
            h = ppool.hash_block(0, toks)
            a.cache_block(p, h, toks)
            b.cache_block(p, h, toks)
        elif op < 0.95:
            toks = rng.choice(pages_of_tokens)
            h = ppool.hash_block(0, toks)
            got = a.get_cached_block(h, toks)
            assert got == b.get_cached_block(h, toks)
            if got >= 0 and rng.random() < 0.5:
                a.touch(got)
                b.touch(got)
                held.append(got)
        else:
            assert a.reset_prefix_cache() == b.reset_prefix_cache()
        assert a.free_list() == b.free_list() and a.num_free == b.num_free and a.num_cached == b.num_cached
        assert list(a.ref) == b.ref and list(a.hash) == b.hash and a.evictions == b.evictions
        a.check_invariants()
    if a.num_free:
        with pytest.raises(PoolError, match="double free"):
            a.free_blocks([a.free_list()[0]])


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 10])
def test_cache_manager_matches_the_plain_manager(seed, window):
    rng = random.Random(100 + seed)
    bs = 4
    groups = [("full", None, 24)] + ([("win", window, 24)] if window else [])
    a = CacheManager([PageGroup(n, (i,), w, nb) for i, (n, w, nb) in enumerate(groups)], bs, True, 6)
    b = pcache.CacheManager([pcache.PageGroup(n, (i,), w, nb) for i, (n, w, nb) in enumerate(groups)], bs, True, 6)
    live = []
    prefixes = [[rng.randrange(50) for _ in range(12)] for _ in range(2)]

    def same(ra, rb):
        assert ra.tables == rb.tables and ra.hashes == rb.hashes and ra.committed == rb.committed
        assert ra.state_slot == rb.state_slot and ra.state_fresh == rb.state_fresh and ra.epoch == rb.epoch

    for _ in range(400):
        op = rng.random()
        if op < 0.3 and len(live) < 6:
            toks = (rng.choice(prefixes)[:] if rng.random() < 0.6 else []) + [rng.randrange(50) for _ in range(rng.randrange(1, 30))]
            ra, rb = a.new_request(), b.new_request()
            assert a.allot_state(ra) == b.allot_state(rb)
            a.update_hashes(ra, toks)
            b.update_hashes(rb.hashes, toks)
            na, ta = a.find_cached_prefix(toks, ra.hashes)
            nb_, tb = b.find_cached_prefix(toks, rb.hashes)
            assert (na, ta) == (nb_, tb)
            n_new = min(len(toks) - na, rng.randrange(1, 9))
            ok = a.allocate(ra, na, n_new, ta)
            assert ok == b.allocate(rb, na, n_new, tb)
            if ok:
                live.append([ra, rb, toks, na + n_new])
                a.commit(ra, toks, na + n_new)
                b.commit(rb, toks, na + n_new)
            else:
                a.free(ra)
                b.free(rb)
            same(ra, rb)
        elif op < 0.8 and live:
            ent = rng.choice(live)
            ra, rb, toks, done = ent
            if done == len(toks):
                toks.append(rng.randrange(50))
            n_new = min(len(toks) - done, rng.randrange(1, 7))
            ok = a.allocate(ra, done, n_new)
            assert ok == b.allocate(rb, done, n_new)
            if ok:
                ent[3] = done + n_new
                a.update_hashes(ra, toks)
                b.update_hashes(rb.hashes, toks)
                a.commit(ra, toks, ent[3])
                b.commit(rb, toks, ent[3])
                assert a.slot_of(ra, 0, ent[3] - 1) == b.slot_of(rb, 0, ent[3] - 1)
            else:
                a.free(ra)
                b.free(rb)
                live.remove(ent)
            same(ra, rb)
        elif live:
            ent = rng.choice(live)
            a.free(ent[0])
            b.free(ent[1])
            same(ent[0], ent[1])
            live.remove(ent)
        for g in range(len(groups)):
            assert a.pools[g].free_list() == b.pools[g].free_list() and list(a.pools[g].ref) == b.pools[g].ref
        assert a.slots.num_free == b.slots.num_free and abs(a.usage - b.usage) < 1e-12
        a.check_invariants()


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("policy", ["fcfs", "priority"])
def test_scheduler_matches_the_plain_scheduler(seed, policy):
    """Random arrivals, few pages (so that requests are preempted), prefix sharing, finishing at random: every
    step both schedulers pick the same requests with the same portions and preempt the same ones."""
    rng = random.Random(1000 + seed)
    bs = 4
    cfg = dict(max_num_seqs=4, max_num_batched_tokens=rng.choice([8, 16, 64]), policy=policy,
               long_prefill_token_threshold=rng.choice([0, 0, 5]), enable_chunked_prefill=rng.random() < 0.8)
    ca = CacheManager([PageGroup("full", (0,), None, 14)], bs, True, 4)
    cb = pcache.CacheManager([pcache.PageGroup("full", (0,), None, 14)], bs, True, 4)
    sa, sb = Scheduler(SchedulerConfig(**cfg), ca), psched.Scheduler(SchedulerConfig(**cfg), cb)
    prefix = [rng.randrange(30) for _ in range(8)]
    reqs = {}
    next_id = 0
    n_preempted = 0
    for step in range(300):
        if rng.random() < 0.25 and len(reqs) < 7:
            toks = (prefix[:] if rng.random() < 0.5 else []) + [rng.randrange(30) for _ in range(rng.randrange(1, 22))]
            prio = rng.randrange(3)
            ra = Request(id=next_id, tokens=toks, n_prompt=len(toks), params=SamplingParams(), priority=prio, arrival=float(step))
            rb = psched.Request(id=next_id, tokens=list(toks), priority=prio, arrival=float(step))
            sa.add_request(ra)
            sb.add_request(rb)
            reqs[next_id] = (ra, rb)
            next_id += 1
        oa, ob = sa.schedule(), sb.schedule()
        assert [(s.req.id, s.n_new_tokens, s.resumed) for s in oa.scheduled] == [(s.req.id, s.n_new_tokens, s.resumed) for s in ob.scheduled]
        assert [r.id for r in oa.preempted] == [r.id for r in ob.preempted] and oa.total_tokens == ob.total_tokens
        n_preempted += len(oa.preempted)
        sa.update_after_step(oa)
        sb.update_after_step(ob)
        for s in oa.scheduled:
            ra, rb = reqs[s.req.id]
            if ra.num_computed_tokens == ra.n_tokens:          # the step reached the request's end: a token is sampled
                t = rng.randrange(30)
                ra.tokens.append(t)
                rb.tokens.append(t)
        for rid in list(reqs):
            ra, rb = reqs[rid]
            assert (ra.status, ra.num_computed_tokens, ra.num_cached_tokens, ra.num_preemptions) == \
                (rb.status, rb.num_computed_tokens, rb.num_cached_tokens, rb.num_preemptions)
            if rb.cache is not None:
                assert ra.cache.tables == rb.cache.tables and ra.cache.hashes == rb.cache.hashes
            if rng.random() < 0.04 or ra.n_tokens > 60:
                from iian_b200.engine.request import RequestStatus
                sa.finish_request(ra, RequestStatus.FINISHED_STOPPED)
                sb.finish_request(rb, RequestStatus.FINISHED_STOPPED)
                del reqs[rid]
        assert [r.id for r in sa.waiting] == [r.id for r in sb.waiting] and [r.id for r in sa.running] == [r.id for r in sb.running]
        assert ca.pools[0].free_list() == cb.pools[0].free_list()
        assert sa.num_preemptions == sb.num_preemptions and ca.prefix_hits == cb.prefix_hits and ca.prefix_queries == cb.prefix_queries
        ca.check_invariants()
    assert sa.has_requests == sb.has_requests
