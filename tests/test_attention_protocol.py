"""Host-side model of the barrier protocols of the two pipelined attention kernels (no GPU needed).

`csrc/attention/attn_fwd_dual.cu` and `csrc/attention/attn_bwd_pipe.cu` each run four or five sequential roles (loader, MMA issuers,
softmax groups) that meet only on mbarriers.  The roles are transcribed here as generators over the same barriers with the
hardware's phase-parity semantics, asynchronous work (TMA copies, tcgen05 products) completes after a random delay, in order per
issuing thread, and a random scheduler interleaves the roles.  The model checks, for every tile geometry the launchers can
produce, that every role finishes (no wait can stay unsatisfied: on the GPU that would be a bounded wait giving up), and that
no buffer is overwritten while a product that reads it is still in flight or before its consumer has taken it.
"""
import random

import pytest


class Barrier:
    """mbarrier: `count` arrivals complete a phase; `done(parity)` is try_wait.parity (true once the phase of that parity is over)."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def done(self, parity):
        return (self.phase & 1) != (parity & 1)


class AsyncQueue:
    """Work issued to an asynchronous unit by one thread: items complete in issue order after a random delay; an item is a
    callable run at completion (a commit's arrival, a copy's arrival, releasing a read lock)."""

    def __init__(self, rng, max_delay):
        self.rng, self.max_delay, self.items = rng, max_delay, []

    def push(self, fn):
        self.items.append([self.rng.randint(0, self.max_delay), fn])

    def tick(self):
        if self.items:
            if self.items[0][0] <= 0:
                self.items.pop(0)[1]()
                return True
            self.items[0][0] -= 1
        return False


def run(roles, queues, rng, limit=400000, starved=None, starve=0.0):
    """Random interleaving of the role generators; each yields (barrier, parity) to wait or None to be rescheduled.
    `starved`: a role that is skipped with probability `starve` each round (a thread that is slow to notice its barrier)."""
    waiting = {name: None for name in roles}
    live = dict(roles)
    for _ in range(limit):
        if not live and not any(q.items for q in queues):
            return
        for q in queues:
            q.tick()
        names = list(live)
        rng.shuffle(names)
        for name in names:
            if name == starved and rng.random() < starve:
                continue
            cond = waiting[name]
            if cond is not None and not cond[0].done(cond[1]):
                continue
            try:
                waiting[name] = next(live[name])
            except StopIteration:
                del live[name]
                waiting[name] = None
    stuck = {n: (id(w[0]), w[1]) for n, w in waiting.items() if n in live and w is not None}
    raise AssertionError(f"roles never finished: {sorted(live)} waiting on {stuck}")


# ---- forward: two query tiles per CTA -------------------------------------------------------------------------------------------

def forward_dual(q0, window, seq_len, rng, max_delay, stages=4, starved=None):
    tile = 128
    first_a, first_b = q0 - window, q0 + tile - window
    lo_a, lo_b = (first_a // tile if first_a > 0 else 0), (first_b // tile if first_b > 0 else 0)
    hi_a = q0 // tile
    total = hi_a + 1 - lo_a + 1
    n = [hi_a - lo_a + 1, hi_a + 1 - lo_b + 1]
    u0 = [0, lo_b - lo_a]
    bar_q = Barrier(1)
    bar_s, bar_p, bar_o = [Barrier(1), Barrier(1)], [Barrier(1), Barrier(1)], [Barrier(1), Barrier(1)]      # bar_p: the 128 threads as one
    bar_full, bar_free = [Barrier(1) for _ in range(stages)], [Barrier(2) for _ in range(stages)]
    tma, mma = AsyncQueue(rng, max_delay), [AsyncQueue(rng, max_delay), AsyncQueue(rng, max_delay)]
    stage_tile = [None] * stages           # key/value tile a stage holds (None while a copy is in flight)
    readers = [0] * stages                 # products in flight that read the stage
    s_owner = ["free", "free"]             # S_x columns: free -> product in flight -> ready for the softmax -> free
    p_ready = [False, False]
    finished = []

    def loader():
        tma.push(bar_q.arrive)
        for u in range(total):
            st, use = u % stages, u // stages
            if use > 0:
                yield bar_free[st], use - 1
            assert readers[st] == 0, "a stage is refilled while a product still reads it"
            stage_tile[st] = None

            def landed(st=st, u=u):
                stage_tile[st] = u
                bar_full[st].arrive()
            tma.push(landed)
        finished.append("loader")

    def issuer(x):
        def issue_s(u):
            st = u % stages
            yield bar_full[st], u // stages
            assert stage_tile[st] == u, "S reads a stage that does not hold its key tile"
            assert s_owner[x] == "free", "S overwrites scores the softmax has not consumed"
            s_owner[x] = "mma"
            readers[st] += 1

            def done(st=st):
                readers[st] -= 1
                s_owner[x] = "ready"
                bar_s[x].arrive()
            mma[x].push(done)

        yield bar_q, 0
        yield from issue_s(u0[x])
        for i in range(n[x]):
            yield bar_p[x], i
            assert p_ready[x], "PV issued before P was written"
            p_ready[x] = False
            st = (u0[x] + i) % stages
            assert stage_tile[st] == u0[x] + i, "PV reads a stage that does not hold its value tile"
            readers[st] += 1
            last = i + 1 == n[x]

            def pv_done(st=st, last=last):
                readers[st] -= 1
                if last:
                    bar_o[x].arrive()
            mma[x].push(pv_done)
            if not last:
                yield from issue_s(u0[x] + i + 1)
        finished.append(f"issuer{x}")

    def softmax(x):
        lo_x = lo_a if x == 0 else lo_b
        for i in range(n[x]):
            yield bar_s[x], i
            assert s_owner[x] == "ready"
            if i > 0:
                done = lo_x + i - 1
                fb = bar_free[(done - lo_a) % stages]
                fb.arrive()
                if (done < lo_b) if x == 0 else (done > hi_a):
                    fb.arrive()
            yield None                                 # the arithmetic: other roles run meanwhile
            s_owner[x] = "free"
            p_ready[x] = True
            bar_p[x].arrive()
        yield bar_o[x], 0
        finished.append(f"softmax{x}")

    roles = {"loader": loader(), "issuer0": issuer(0), "issuer1": issuer(1), "softmax0": softmax(0), "softmax1": softmax(1)}
    run(roles, [tma] + mma, rng, starved=starved, starve=0.95)
    assert len(finished) == 5


@pytest.mark.parametrize("seq_len,window", [(256, 0), (256, 1000), (512, 128), (768, 77), (1024, 300), (2048, 1024), (2048, 1000), (2048, 5000),
                                            (4096, 4096), (4096, 129)])
@pytest.mark.parametrize("max_delay", [0, 3, 40])
def test_forward_with_two_query_tiles_never_stalls_and_never_reuses_a_live_buffer(seq_len, window, max_delay):
    rng = random.Random(seq_len * 131 + window * 7 + max_delay)
    for q0 in range(0, seq_len, 256):
        for _ in range(3):
            forward_dual(q0, min(window, seq_len), seq_len, rng, max_delay)


def test_forward_model_notices_a_ring_that_is_too_shallow():
    """The check has teeth: a ring of one stage cannot serve two query tiles that are one key tile apart (a stage is released only
    when both have finished with it, and the tile ahead needs the next key tile first); the model reports it (as the stall that the kernel would
    report through its status word, or as a product reading a stage that holds another tile).  Two stages already suffice for progress; the kernel uses four for prefetch."""
    with pytest.raises(AssertionError):                # a stall, or a product that finds the wrong tile in the only stage
        forward_dual(1280, 1024, 2048, random.Random(0), 3, stages=1)
    for seed in range(10):
        forward_dual(1280, 1024, 2048, random.Random(seed), 3, stages=2)


# ---- backward: score products of the next query tile ahead of the gradient products ------------------------------------------------

def backward_pipe(n_iter, rng, max_delay, stages=3, starved=None):
    bar_kv, bar_sdp, bar_sread, bar_pds, bar_mma = Barrier(1), Barrier(1), Barrier(1), Barrier(1), Barrier(1)   # 256-thread barriers as one
    bar_qdo = [Barrier(1) for _ in range(stages)]
    tma, mma_s, mma_g = AsyncQueue(rng, max_delay), AsyncQueue(rng, max_delay), AsyncQueue(rng, max_delay)
    stage_iter = [None] * stages
    readers = [0] * stages
    sdp = {"state": "free"}               # S / dP columns of TMEM
    pds = {"holds": None, "readers": 0}   # P / dS tiles in shared memory
    dq = {"holds": None}                  # dQ columns of TMEM
    drained = []
    finished = []

    def loader():
        tma.push(bar_kv.arrive)

        def load(it):
            st = it % stages
            assert readers[st] == 0, "a Q/dO stage is refilled while a product still reads it"
            stage_iter[st] = None

            def landed(st=st, it=it):
                stage_iter[st] = it
                bar_qdo[st].arrive()
            tma.push(landed)
        for it in range(min(stages, n_iter)):
            load(it)
        for it in range(stages, n_iter):
            yield bar_mma, it - stages
            load(it)
        finished.append("loader")

    def issue_sdp(it):
        st = it % stages
        yield bar_qdo[st], it // stages
        assert stage_iter[st] == it
        assert sdp["state"] == "free", "S/dP overwritten before the softmax warps have read them"
        sdp["state"] = "mma"
        readers[st] += 1

        def done(st=st):
            readers[st] -= 1
            sdp["state"] = "ready"
            bar_sdp.arrive()
        mma_s.push(done)

    def score_issuer():
        yield bar_kv, 0
        if n_iter > 0:
            yield from issue_sdp(0)
        for it in range(n_iter - 1):
            yield bar_sread, it
            yield from issue_sdp(it + 1)
        finished.append("score_issuer")

    def gradient_issuer():
        yield bar_kv, 0
        for it in range(n_iter):
            st = it % stages
            yield bar_pds, it
            yield bar_qdo[st], it // stages
            assert stage_iter[st] == it and pds["holds"] == it
            assert dq["holds"] is None, "dQ overwritten before the previous tile's dQ was drained"
            readers[st] += 1
            pds["readers"] += 1
            dq["holds"] = ("mma", it)

            def done(st=st, it=it):
                readers[st] -= 1
                pds["readers"] -= 1
                dq["holds"] = it
                bar_mma.arrive()
            mma_g.push(done)
        finished.append("gradient_issuer")

    def softmax():
        def drain(jt):
            yield bar_mma, jt
            assert dq["holds"] == jt
            dq["holds"] = None
            drained.append(jt)
        for it in range(n_iter):
            yield bar_sdp, it
            assert sdp["state"] == "ready"
            yield None                                 # P and dS formed in registers
            sdp["state"] = "free"
            bar_sread.arrive()
            if it > 0:
                yield from drain(it - 1)
            assert pds["readers"] == 0, "P/dS stored while the previous gradient products still read the tiles"
            pds["holds"] = it
            bar_pds.arrive()
        if n_iter > 0:
            yield from drain(n_iter - 1)
        finished.append("softmax")

    roles = {"loader": loader(), "score_issuer": score_issuer(), "gradient_issuer": gradient_issuer(), "softmax": softmax()}
    run(roles, [tma, mma_s, mma_g], rng, starved=starved, starve=0.95)
    assert len(finished) == 4 and drained == list(range(n_iter))


@pytest.mark.parametrize("n_iter", [1, 2, 3, 4, 5, 9, 18, 36])
@pytest.mark.parametrize("max_delay", [0, 3, 40])
def test_pipelined_backward_never_stalls_and_never_reuses_a_live_buffer(n_iter, max_delay):
    rng = random.Random(n_iter * 17 + max_delay)
    for _ in range(5):
        backward_pipe(n_iter, rng, max_delay)


@pytest.mark.parametrize("starved", ["loader", "issuer0", "issuer1", "softmax0", "softmax1"])
def test_forward_protocol_survives_a_role_that_lags_far_behind(starved):
    """A role that notices its barriers late (so that a barrier it waits on may have moved on by more than one phase where the
    protocol allows that) only delays the others; parity tests never mistake a later phase for an earlier one."""
    rng = random.Random(sum(map(ord, starved)))
    for q0 in (0, 256, 1280, 1792):
        forward_dual(q0, 1024, 2048, rng, 5, starved=starved)


@pytest.mark.parametrize("starved", ["loader", "score_issuer", "gradient_issuer", "softmax"])
def test_backward_protocol_survives_a_role_that_lags_far_behind(starved):
    rng = random.Random(sum(map(ord, starved)))
    for n_iter in (1, 3, 4, 9, 18):
        backward_pipe(n_iter, rng, 5, starved=starved)
