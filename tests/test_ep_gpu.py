"""Expert parallelism on real GPUs (2 ranks, one per GPU, NCCL with NVLS off): hp_ep_init, a batched pass and lock-step
fused rounds on a reduced MoE model must reproduce the single-GPU results bit for bit on every rank. Skipped when fewer
than two GPUs are visible."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
pytestmark = pytest.mark.gpu


def _run(eng, cfg):
    S, n = 4, 2
    prompts = [[int(x) for x in np.random.default_rng(70 + s).integers(0, cfg.n_vocab, size=6 + s)] for s in range(S)]
    for s in range(S):
        eng.prefill(s, prompts[s], with_mtp=True)
        eng.spec_begin(s, int(eng.topk(0, 1)[0][0]), len(prompts[s]), eng.h_nextn_ptr())
    outs = [[] for _ in range(S)]
    for r in range(3):
        got = eng.spec_round_slots(list(range(S)), n, [[-1, (11 * r + s) % cfg.n_vocab] for s in range(S)])
        for s in range(S):
            outs[s] += got[s]
    eng.forward([(s, [3 + s, 400 + s, 9], 40) for s in range(S)])
    return outs, eng.logits(3 * S).copy()


def _worker(rank, world, port, out, nccl_only=False):
    if nccl_only:
        os.environ["HIPSTER_B200_EP_NCCL"] = "1"
    import faulthandler
    faulthandler.dump_traceback_later(240, exit=True)      # a rank that waits for a lost peer must not outlive the test
    try:
        _worker_body(rank, world, port, out, nccl_only)
    except Exception as e:                                  # report instead of leaving the peer to wait
        out[rank] = ("error", repr(e))
        os._exit(1)
    os._exit(0)                                             # skip interpreter teardown (a process group without its peer can block there)


def _worker_body(rank, world, port, out, nccl_only=False):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    import hipster_b200 as hb
    from hipster_b200 import ep
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    cfg = hb.ModelCfg.preset("tiny-moe", ep_rank=rank, ep_world=world)
    eng = hb.Engine(cfg)
    eng.ep_init(ep.broadcast_unique_id(dist, rank))
    peer = eng.ep_peer()
    outs, logits = _run(eng, cfg)
    eng.close()
    solo_cfg = hb.ModelCfg.preset("tiny-moe")
    solo = hb.Engine(solo_cfg)
    want_outs, want_logits = _run(solo, solo_cfg)
    solo.close()
    out[rank] = (outs == want_outs, bool(np.array_equal(logits.view(np.uint32), want_logits.view(np.uint32))), peer)
    dist.barrier()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("nccl_only", [False, True])
def test_expert_parallel_two_gpus_bit_exact_vs_single_gpu(nccl_only):
    """Both forms of the exchange: over peer memory (the default for one process per GPU on one node; the fused rounds
    are single graphs) and as the NCCL collective (HIPSTER_B200_EP_NCCL)."""
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager(); out = mgr.dict()
    port = 32500 + (os.getpid() % 2000) + (7 if nccl_only else 0)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out, nccl_only), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    alive = [p.is_alive() for p in procs]
    for p in procs:
        if p.is_alive():
            p.kill()
    assert not any(alive), f"a rank did not finish: {dict(out)}"
    assert all(p.exitcode == 0 for p in procs), dict(out)
    assert out[0] == (True, True, not nccl_only) and out[1] == (True, True, not nccl_only), dict(out)
