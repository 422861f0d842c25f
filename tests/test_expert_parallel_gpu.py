"""GPU, 2 / 4 / 8 ranks over NCCL (as many as are visible): expert-parallel ``grouped_gemm_fp8`` against the single-GPU op on the
same routed rows.  Forward output and activation gradient must be bit-identical (1x128 row scales
and each output row do not depend on which other rows share a tile); weight gradients are compared
within the GEMM gate because the 128-row column blocks are composed differently.
Three forms are covered: the serial chain of autograd nodes over NCCL all-to-alls, the single node that
overlaps the weight quantisation and wgrad with the exchanges, and the peer-memory exchange that writes
rows straight into the owners' buffers (same results bit for bit in out and grad_a).
Cases that need more GPUs than are visible are skipped."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

E, K, N = 8, 512, 384


def _data(WORLD):
    g = torch.Generator().manual_seed(5)
    counts = torch.randint(0, 200, (WORLD, E), generator=g)
    counts[:, 3] = 0
    xs = [torch.randn(int(counts[r].sum()), K, generator=g).to(torch.bfloat16) for r in range(WORLD)]
    gos = [(torch.randn(int(counts[r].sum()), N, generator=g) * 1e-3).to(torch.bfloat16) for r in range(WORLD)]
    w = (torch.randn(E, N, K, generator=g) * 0.02).to(torch.bfloat16)
    return counts, xs, gos, w


def _worker(rank, store_path, q, overlap, WORLD):
    torch.cuda.set_device(rank)
    # a rank that fails leaves while the others still hold the communicator: keep NVLink multicast objects out of it
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    store = dist.FileStore(store_path, WORLD)
    dist.init_process_group("nccl", store=store, rank=rank, world_size=WORLD, device_id=torch.device("cuda", rank))
    try:
        from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, ScalingGranularity
        from primus_turbo_b200.pytorch.dist.expert_parallel import ep_grouped_gemm_fp8

        cfg = Float8QuantConfig(granularity=ScalingGranularity.BLOCKWISE, block_size=128)
        counts, xs, gos, w = _data(WORLD)
        e_loc = E // WORLD
        x = xs[rank].cuda().requires_grad_(True)
        w_loc = w[rank * e_loc : (rank + 1) * e_loc].cuda().requires_grad_(True)
        if overlap in ("peer", "peer-collective"):
            # rows written straight into the owners' IPC-mapped buffers, two steps (regions are reused)
            from primus_turbo_b200.pytorch.dist.expert_parallel import build_peer_plan, expert_parallel_apply_peer
            from primus_turbo_b200.pytorch.dist.peer_exchange import PeerExchange
            from primus_turbo_b200.pytorch.ops import grouped_gemm_fp8

            host_group = dist.new_group(backend="gloo")
            ex = PeerExchange(None, host_group, torch.device("cuda", rank), capacity_rows=int(counts.sum()),
                              local_rows=int(counts.sum(1).max()),
                              ordering="collective" if overlap == "peer-collective" else None)
            assert ex.ordering == ("collective" if overlap == "peer-collective" else "flags")
            for _ in range(2):
                x.grad = w_loc.grad = None
                plan = build_peer_plan(counts[rank], host_group, torch.device("cuda", rank))
                out = expert_parallel_apply_peer(
                    x, lambda rows, lens: grouped_gemm_fp8(rows, w_loc, lens, config=cfg), ex, plan)
                out.backward(gos[rank].cuda())
            torch.cuda.synchronize()
            from primus_turbo_b200 import _lib

            assert _lib.copy_segments_status() == 0
        else:
            out = ep_grouped_gemm_fp8(x, w_loc, counts[rank].cuda(), config=cfg, overlap=overlap)
            out.backward(gos[rank].cuda())
            torch.cuda.synchronize()
        q.put((rank, out.detach().float().cpu().tolist(), x.grad.float().cpu().tolist(), w_loc.grad.float().cpu().tolist()))
        dist.barrier()
        if overlap in ("peer", "peer-collective"):
            ex.close()
    except Exception as exc:
        q.put((rank, repr(exc), None, None))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("overlap", [False, True, "peer", "peer-collective"])
@pytest.mark.parametrize("WORLD", [2, 4, 8])
def test_expert_parallel_matches_single_gpu(overlap, WORLD):
    if torch.cuda.device_count() < WORLD:
        pytest.skip(f"needs {WORLD} GPUs")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker, args=(r, os.path.join(d, "store"), q, overlap, WORLD)) for r in range(WORLD)]
        for p in procs:
            p.start()
        res = {}
        try:
            for _ in range(WORLD):
                r, out, gx, gw = q.get(timeout=300)
                assert gx is not None, f"rank {r} failed: {out}"
                res[r] = (torch.tensor(out), torch.tensor(gx), torch.tensor(gw))
            for p in procs:
                p.join(timeout=120)
                assert p.exitcode == 0
        finally:
            # after a failure the surviving ranks wait for the one that left: end exactly the children started here
            for p in procs:
                if p.is_alive():
                    p.terminate()
                    p.join(timeout=30)

    from oracle import fp8_oracle as O
    from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, ScalingGranularity
    from primus_turbo_b200.pytorch.ops import grouped_gemm_fp8

    cfg = Float8QuantConfig(granularity=ScalingGranularity.BLOCKWISE, block_size=128)
    counts, xs, gos, w = _data(WORLD)
    # single-GPU evaluation: rows of all ranks, expert-major with the source rank as minor order
    rows, grads, index = [], [], []
    for e in range(E):
        for r in range(WORLD):
            lo = int(counts[r, :e].sum())
            n = int(counts[r, e])
            rows.append(xs[r][lo : lo + n])
            grads.append(gos[r][lo : lo + n])
            index.append((r, lo, n))
    a = torch.cat(rows).cuda().requires_grad_(True)
    wd = w.cuda().requires_grad_(True)
    lens = counts.sum(0).to(torch.int64).cuda()
    out = grouped_gemm_fp8(a, wd, lens, config=cfg)
    out.backward(torch.cat(grads).cuda())
    pos = 0
    for r, lo, n in index:
        assert torch.equal(res[r][0][lo : lo + n], out[pos : pos + n].detach().float().cpu())
        assert torch.equal(res[r][1][lo : lo + n], a.grad[pos : pos + n].float().cpu())
        pos += n
    e_loc = E // WORLD
    for r in range(WORLD):
        ref = wd.grad[r * e_loc : (r + 1) * e_loc].float().cpu()
        assert O.rel_frobenius(ref, res[r][2]) <= 2e-2
