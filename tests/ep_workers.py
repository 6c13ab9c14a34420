"""Worker processes of the expert-parallel tests (spawned with
torch.multiprocessing).  Kept in a module of their own so that spawn can
import them."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _init(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


def split_tokens(T, world):
    """Uneven on purpose: rank r owns rows [starts[r], starts[r+1])."""
    base = T // world
    sizes = [base] * world
    sizes[0] += T - base * world
    if world > 1 and sizes[-1] > 3:
        sizes[-1] -= 3
        sizes[0] += 3
    starts = np.concatenate([[0], np.cumsum(sizes)])
    return starts


# ---------------------------------------------------------------------------
# CPU: the exchange protocol of csrc/ep.cuh restated over gloo, the experts
# computed by the oracle.  Checks the host-side plan (moe_b200_ep_plan), the
# regroup-by-expert indexing and the return path against a single-process run.


def cpu_worker(rank, world, port, shape_kw, T, seed, outdir):
    import gpt_oss_amd_b200 as pkg
    from gpt_oss_amd_b200 import capi, synth
    from oracle import oracle

    _init(rank, world, port)
    shape = pkg.MoEShape(**shape_kw)
    H, E, K = shape.hidden, shape.n_experts, shape.top_k
    first, n_local = capi.shard_range(E, world, rank)
    lw = synth.make_layer(shape, seed, first=first, n=n_local)
    starts = split_tokens(T, world)
    x = synth.bf16_bits_to_f32(synth.make_tokens(T, H, seed))[starts[rank]:starts[rank + 1]]
    wr = synth.bf16_bits_to_f32(lw.w_router)
    _, ti, tw = oracle.route(x, wr, lw.b_router, K, round_mode=1)
    Tl = x.shape[0]
    # rows sorted by global expert, token order inside an expert (permute_kernel)
    flat_e = ti.reshape(-1)
    order = np.argsort(flat_e, kind="stable")
    slot_of = np.empty(Tl * K, dtype=np.int64)
    slot_of[order] = np.arange(Tl * K)
    xs = x[order // K]
    cnt = np.bincount(flat_e, minlength=E).astype(np.int32)
    # all-gather of counts, host plan
    gathered = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(cnt))
    cnt_all = np.stack([g.numpy() for g in gathered])
    send_cnt, send_off, recv_cnt, recv_off = capi.ep_plan(E, world, rank, cnt_all)
    # dispatch
    xrecv = torch.zeros(sum(recv_cnt), H)
    reqs = []
    for p in range(world):
        if p == rank:  # gloo has no self-send: local copy (NCCL handles it inside a group)
            xrecv[recv_off[p]:recv_off[p] + recv_cnt[p]] = torch.from_numpy(
                xs[send_off[p]:send_off[p] + send_cnt[p]])
            continue
        if send_cnt[p]:
            reqs.append(dist.isend(torch.from_numpy(np.ascontiguousarray(
                xs[send_off[p]:send_off[p] + send_cnt[p]])), p))
        if recv_cnt[p]:
            reqs.append(dist.irecv(xrecv[recv_off[p]:recv_off[p] + recv_cnt[p]], p))
    for r in reqs:
        r.wait()
    xrecv = xrecv.numpy()
    # regroup by local expert (regroup_plan_kernel / regroup_index_kernel)
    g_cnt = cnt_all[:, first:first + n_local].sum(axis=0)
    g_off = np.concatenate([[0], np.cumsum(g_cnt)])
    gather_src = np.empty(int(g_off[-1]), dtype=np.int64)
    for le in range(n_local):
        for p in range(world):
            n = int(cnt_all[p, first + le])
            src = recv_off[p] + int(cnt_all[p, first:first + le].sum())
            dst = int(g_off[le]) + int(cnt_all[:p, first + le].sum())
            gather_src[dst:dst + n] = np.arange(src, src + n)
    xgrp = xrecv[gather_src]
    cache = oracle.ExpertCache(lw.blocks1, lw.scales1, lw.bias1, lw.blocks2, lw.scales2, lw.bias2,
                               first_expert=first)
    ysend = np.zeros((len(gather_src), H), dtype=np.float32)
    for le in range(n_local):
        a, b = int(g_off[le]), int(g_off[le + 1])
        if b > a:
            e = first + le
            y = oracle.expert_rows(xgrp[a:b], cache.w1(e), cache.bias1(e), cache.w2(e), cache.bias2(e),
                                   round_mode=1)
            ysend[gather_src[a:b]] = y  # GEMM2 writes rows back in received order (row_dst)
    # return
    yrecv = torch.zeros(Tl * K, H)
    reqs = []
    for p in range(world):
        if p == rank:
            yrecv[send_off[p]:send_off[p] + send_cnt[p]] = torch.from_numpy(
                ysend[recv_off[p]:recv_off[p] + recv_cnt[p]])
            continue
        if recv_cnt[p]:
            reqs.append(dist.isend(torch.from_numpy(np.ascontiguousarray(
                ysend[recv_off[p]:recv_off[p] + recv_cnt[p]])), p))
        if send_cnt[p]:
            reqs.append(dist.irecv(yrecv[send_off[p]:send_off[p] + send_cnt[p]], p))
    for r in reqs:
        r.wait()
    yrecv = yrecv.numpy()
    # combine: ascending expert order (combine_kernel)
    out = np.zeros((Tl, H), dtype=np.float32)
    for t in range(Tl):
        for k in np.argsort(ti[t]):
            out[t] += yrecv[slot_of[t * K + k]] * tw[t, k]
    np.savez(os.path.join(outdir, f"cpu_rank{rank}.npz"), out=out, topk_i=ti, topk_w=tw,
             start=starts[rank])
    dist.barrier()
    dist.destroy_process_group()


# ---------------------------------------------------------------------------
# GPU: the real thing, one process per GPU; the exchange inside the library
# over NCCL (mode "nccl") or over peer memory (mode "peer").


def gpu_worker(rank, world, port, shape_kw, T, seed, outdir, gemm_impl, mode, sample=0):
    """One rank of an expert-parallel run.  With ``sample`` > 0 (full-size layers) the
    rank itself checks that many of its own tokens against the CPU oracle -- experts
    are regenerated from the seed, whichever rank holds them -- and saves the figures."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import json

    import gpt_oss_amd_b200 as pkg
    from gpt_oss_amd_b200 import synth
    from oracle import parity

    _init(rank, world, port)
    torch.cuda.set_device(rank)
    shape = pkg.MoEShape(**shape_kw)
    starts = split_tokens(T, world)
    Tl = int(starts[rank + 1] - starts[rank])
    eng = pkg.MoEEngine(shape, max_tokens=max(int(np.diff(starts).max()), 1), ep_rank=rank,
                        ep_size=world, device=rank, gemm_impl=gemm_impl)
    eng.ep_connect(dist, mode)
    lw = synth.make_layer(shape, seed, first=eng.first_expert, n=eng.n_local)
    eng.load_layer(0, lw)
    x_bits = synth.make_tokens(T, shape.hidden, seed)[starts[rank]:starts[rank + 1]]
    t = torch.from_numpy(np.ascontiguousarray(x_bits).view(np.int16)).cuda().view(torch.bfloat16)
    out, sc, ti, tw = eng.forward(0, t, side=True)
    torch.cuda.synchronize()
    counts = eng.last_expert_counts()
    # second call: the last rank brings no tokens at all
    t2 = t if rank != world - 1 else t[:0]
    out2 = eng.forward(0, t2)
    torch.cuda.synchronize()
    # third call: everybody again (the call after a rank had nothing to send)
    out3 = eng.forward(0, t)
    torch.cuda.synchronize()
    status = eng.device_status()
    figures = {}
    if sample > 0 and Tl > 0:
        rows = np.unique(np.linspace(0, Tl - 1, sample).astype(np.int64))
        res = {"out": out.cpu().numpy()[rows], "topk_i": ti.cpu().numpy()[rows],
               "topk_w": tw.cpu().numpy()[rows]}
        figures = parity.compare_sampled(res, x_bits[rows], lw.w_router, lw.b_router,
                                         lambda e: synth.make_experts(shape, seed, e, 1), shape.top_k)
    np.savez(os.path.join(outdir, f"gpu_rank{rank}.npz"), out=out.cpu().numpy(),
             topk_i=ti.cpu().numpy(), topk_w=tw.cpu().numpy(), out2=out2.cpu().numpy(),
             out3=out3.cpu().numpy(), start=starts[rank], status=status, counts=np.array(counts),
             figures=json.dumps(figures), device_bytes=eng.device_bytes())
    dist.barrier()
    eng.close()
    dist.destroy_process_group()


def gpu_missing_rank_worker(rank, world, port, shape_kw, T, seed, outdir):
    """Failure detection without a GPU fault: rank 1 never joins the first call.  Rank
    0's peer-flag waits run out (2 s), its kernels return, the status word names the
    wait and the context stays usable.  Rank 1 stays alive (its buffers stay mapped)
    until rank 0 has read the status.  Then the ranks agree on a sequence number over
    the host channel, resynchronise, and make a call together that must be right."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import gpt_oss_amd_b200 as pkg
    from gpt_oss_amd_b200 import synth

    _init(rank, world, port)
    torch.cuda.set_device(rank)
    shape = pkg.MoEShape(**shape_kw)
    starts = split_tokens(T, world)
    eng = pkg.MoEEngine(shape, max_tokens=T, ep_rank=rank, ep_size=world, device=rank)
    eng.ep_connect(dist, "peer")
    lw = synth.make_layer(shape, seed, first=eng.first_expert, n=eng.n_local)
    eng.load_layer(0, lw)
    dist.barrier()
    x_all = synth.make_tokens(T, shape.hidden, seed)
    x_bits = x_all[starts[rank]:starts[rank + 1]]
    t = torch.from_numpy(np.ascontiguousarray(x_bits).view(np.int16)).cuda().view(torch.bfloat16)
    status, usable = 0, True
    if rank == 0:
        eng.forward(0, t)
        torch.cuda.synchronize()
        status = eng.device_status()  # reads and clears
        # the context still works
        usable = bool((torch.ones(8, device="cuda") * 2).sum().item() == 16.0)
    dist.barrier()  # nothing is in flight on either rank here
    seqs = [None] * world
    dist.all_gather_object(seqs, eng.ep_peer_sequence())
    eng.ep_peer_resync(max(seqs))
    dist.barrier()
    out, _, ti, tw = eng.forward(0, t, side=True)
    torch.cuda.synchronize()
    status_after = eng.device_status()
    np.savez(os.path.join(outdir, f"miss_rank{rank}.npz"), status=status, usable=usable,
             status_after=status_after, seqs=np.array(seqs), out=out.cpu().numpy(),
             topk_i=ti.cpu().numpy(), topk_w=tw.cpu().numpy())
    dist.barrier()  # a rank leaves only after the other is done, nothing in flight
    eng.close()
    dist.destroy_process_group()
