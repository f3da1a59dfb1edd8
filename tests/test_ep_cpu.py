"""Expert-parallel exchange logic on CPU with two gloo ranks: each rank computes the per-(row, slot) expert outputs of
the experts it owns (exact zeros for the others; the shared expert on rank 0 only), the buffers are summed with an
all-reduce, and the combine runs in slot order. The result must equal the single-rank MoE output bit for bit
(every element has exactly one non-zero contributor, so the summation order cannot matter)."""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _moe_single(orc, W, x, R, E, H, F, k):
    """single-rank restatement: router -> route -> experts -> in-order combine (qwen4exp.cpp:345-354)."""
    L = orc.lib(); P = orc.P
    q, d, s = orc.quantize_x_q8(x)
    lg = np.empty((R, E + 1), np.float32); L.orc_router_gemv(P(W["router"]), P(x), P(lg), E + 1, H, R)
    ids = np.empty((R, k + 1), np.int32); w = np.empty((R, k + 1), np.float32); L.orc_moe_route(P(lg), P(ids), P(w), R, E, k)
    eb_up = 2 * F * (H // 256) * 144; eb_dn = H * (F // 256) * 144
    v = np.zeros((R, k + 1, H), np.float32)
    for t in range(R):
        for e in range(k + 1):
            i = int(ids[t, e])
            Wu = W["up"][i * eb_up:(i + 1) * eb_up] if i >= 0 else W["sh_up"]
            Wd = W["dn"][i * eb_dn:(i + 1) * eb_dn] if i >= 0 else W["sh_dn"]
            gu = np.empty(2 * F, np.float32)
            L.orc_gemv_q4k_q8_seq(P(np.ascontiguousarray(Wu)), P(np.ascontiguousarray(q[t])), P(np.ascontiguousarray(d[t])), P(np.ascontiguousarray(s[t])), P(gu), 2 * F, H)
            act = np.array([L.orc_silu(float(g)) for g in gu[:F]], np.float32) * gu[F:]
            aq, ad, asum = orc.quantize_x_q8(act[None, :])
            L.orc_gemv_q4k_q8_seq(P(np.ascontiguousarray(Wd)), P(aq), P(ad), P(asum), P(v[t, e]), H, F)
    return ids, w, v


def _combine(w, v):
    R, ns, H = v.shape
    y = np.zeros((R, H), np.float32)
    for t in range(R):
        acc = np.zeros(H, np.float32)
        for e in range(ns):
            acc = _fma_vec(w[t, e], v[t, e], acc)
        y[t] = acc
    return y


def _fma_vec(w, v, acc):
    # exact fused multiply-add per element via float64 (the product of two floats is exact in double; one rounding)
    return (np.float64(w) * v.astype(np.float64) + acc.astype(np.float64)).astype(np.float32)


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import orc
    from hipster_b200 import synth, ep
    R, E, H, F, k = 5, 8, 512, 256, 3
    rng = np.random.default_rng(0)
    W = {"router": (rng.normal(0, 1, size=(E + 1, H)) / np.sqrt(H)).astype(np.float32),
         "up": synth.q4k_matrix(E * 2 * F, H, seed=1).reshape(-1), "dn": synth.q4k_matrix(E * H, F, seed=2).reshape(-1),
         "sh_up": synth.q4k_matrix(2 * F, H, seed=3).reshape(-1), "sh_dn": synth.q4k_matrix(H, F, seed=4).reshape(-1)}
    x = synth.activations(R, H, seed=5)
    ids, w, v = _moe_single(orc, W, x, R, E, H, F, k)
    lo, hi = ep.expert_range(rank, world, E)
    mine = v.copy()
    for t in range(R):
        for e in range(k + 1):
            i = int(ids[t, e])
            owned = (lo <= i < hi) if i >= 0 else rank == 0
            if not owned:
                mine[t, e] = 0.0
    buf = torch.from_numpy(mine)
    dist.all_reduce(buf)                       # the exchange: one non-zero contributor per element
    y_ep = _combine(w, buf.numpy())
    y_1 = _combine(w, v)
    ok = np.array_equal(y_ep.view(np.uint32), y_1.view(np.uint32)) and np.array_equal(buf.numpy().view(np.uint32) & 0x7fffffff, v.view(np.uint32) & 0x7fffffff)
    owners = sorted({ep.owner_of(int(i), world, E) for i in ids[ids >= 0]})
    out[rank] = (bool(ok), owners)
    dist.barrier(); dist.destroy_process_group()


def test_expert_parallel_exchange_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager(); out = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert out[0][0] and out[1][0]
    assert out[0][1] == [0, 1]                 # the routing of this input touches experts of both ranks


def test_expert_ranges_partition_the_experts():
    from hipster_b200 import ep
    for world in (1, 2, 4, 8):
        seen = []
        for r in range(world):
            lo, hi = ep.expert_range(r, world, 512)
            seen += list(range(lo, hi))
        assert seen == list(range(512))
        assert ep.owner_of(511, world, 512) == world - 1


def test_owner_rule_of_the_peer_exchange_matches_the_shard_ranges():
    """The device-side rule that decides which rows a rank delivers must agree with the ranges the weights are sharded by."""
    import hipster_b200 as hb
    from hipster_b200 import ep
    L = hb.lib()
    for n_expert in (16, 100, 512):
        for world in range(1, 9):
            for e in range(n_expert):
                assert L.hp_ep_owner(e, n_expert, world) == ep.owner_of(e, world, n_expert), (e, n_expert, world)
            assert L.hp_ep_owner(-1, n_expert, world) == -1 and L.hp_ep_owner(n_expert, n_expert, world) == -1


# ---- the bounded wait of the engine (hp_ep_wait_poll) with host-made failures: no GPU, no NCCL
QUERY = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)


def _poll(query, comm_error, limit_ms):
    import hipster_b200 as hb
    L = hb.lib()
    q = QUERY(query); c = QUERY(comm_error) if comm_error else ctypes.cast(None, QUERY)
    rc = L.hp_ep_wait_poll(q, c, None, limit_ms)
    return rc, L.hp_last_error().decode()


def test_wait_poll_returns_ok_when_the_stream_drains():
    calls = {"n": 0}

    def query(_):
        calls["n"] += 1
        return 0 if calls["n"] >= 4 else 1
    rc, _ = _poll(query, lambda _: 0, 2000)
    assert rc == 0 and calls["n"] == 4


def test_wait_poll_reports_a_communicator_error_as_ecomm():
    rc, msg = _poll(lambda _: 1, lambda _: 3, 2000)          # a fake of ncclCommGetAsyncError returning a failure code
    assert rc == 6 and "asynchronous error 3" in msg
    rc, msg = _poll(lambda _: 9, None, 2000)                 # a fake of cudaStreamQuery returning a failure
    assert rc == 6 and "status 9" in msg


def test_wait_poll_gives_up_after_the_time_limit():
    import time
    t0 = time.perf_counter()
    rc, msg = _poll(lambda _: 1, lambda _: 0, 150)           # the stream never drains: a peer stopped taking part
    dt = time.perf_counter() - t0
    assert rc == 4 and "stopped taking part" in msg and 0.1 < dt < 5.0


def _wait_worker(rank, port, out):
    """Rank 1 leaves without ever posting its contribution; rank 0 waits for it with the engine's bounded wait, its probe
    being "has the peer's message arrived in the store?". The wait must end with a time-out status, not hang."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=2)
    store = dist.distributed_c10d._get_default_store()
    if rank == 1:
        store.set("rank1_alive", "1")        # joins, then exits between steps without posting "contribution"
        dist.destroy_process_group()
        return
    store.wait(["rank1_alive"])

    def query(_):
        return 0 if store.check(["contribution"]) else 1
    rc, msg = _poll(query, lambda _: 0, 400)
    out[0] = (rc, msg)
    dist.destroy_process_group()


def test_wait_poll_times_out_when_a_gloo_peer_leaves():
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager(); out = mgr.dict()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_wait_worker, args=(r, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out[0][0] == 4 and "stopped taking part" in out[0][1]
