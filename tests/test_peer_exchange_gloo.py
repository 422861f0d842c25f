"""CPU: the peer-memory exchange (primus_turbo_b200/pytorch/dist/peer_exchange.py).

* ``segment_tables`` simulated for every rank of 2-, 4- and 8-rank jobs in one process: the dispatch puts
  each row at its expert-major position in its expert's owner, the combine brings it back.
* world sizes 2, 4 and 8 as real processes over gloo (one case with a rank that receives no row at all): regions live in shared memory, published with the same
  handle exchange the GPU path uses, and a copy loop of this test stands in for the device kernel;
  forward and backward against a single-process evaluation, with an expert nobody routes to, and over
  two steps (a region is reused).
* the placement helper.
The host-side row width here is 8 doubles (64 bytes); the GPU tests cover the kernel itself."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from primus_turbo_b200.pytorch.dist.peer_exchange import segment_tables

H = 8
SHAPES = [(2, 6), (4, 8), (8, 16), (4, 4)]  # (4, 4): one expert per rank, so the rank of the unused expert gets no row


def _routing(seed, WORLD, E, step=0):
    g = torch.Generator().manual_seed(seed * 10 + step)
    counts = torch.randint(0, 7, (WORLD, E), generator=g)
    counts[:, 1] = 0  # an expert nobody routes to
    if E > 4:
        counts[1, 4] = 0
    xs = [torch.randn(int(counts[r].sum()), H, generator=g, dtype=torch.float64) for r in range(WORLD)]
    return counts, xs


def _expert_fn(e_global, rows):
    return rows * (e_global + 1.0) + rows.pow(2) * 0.5


def _copy_loop(src, dst_tensors, segs):
    for s, d, n, r in segs.tolist():
        if n:
            dst_tensors[r][d : d + n] = src[s : s + n]


@pytest.mark.parametrize("WORLD,E", SHAPES)
def test_segment_tables_place_every_row(WORLD, E):
    counts, xs = _routing(3, WORLD, E)
    e_loc = E // WORLD
    tabs = [segment_tables(counts, r) for r in range(WORLD)]
    recv = [torch.full((t.rows_out, H), float("nan"), dtype=torch.float64) for t in tabs]
    for r in range(WORLD):
        assert tabs[r].rows_in == xs[r].shape[0]
        assert tabs[r].group_lens.tolist() == counts[:, r * e_loc : (r + 1) * e_loc].sum(0).tolist()
        _copy_loop(xs[r], recv, tabs[r].dispatch)
    for r in range(WORLD):  # expert-major, sources in rank order inside an expert
        want = []
        for e in range(r * e_loc, (r + 1) * e_loc):
            for s in range(WORLD):
                lo = int(counts[s, :e].sum())
                want.append(xs[s][lo : lo + int(counts[s, e])])
        assert torch.equal(recv[r], torch.cat(want) if want else recv[r])
    back = [torch.full_like(x, float("nan")) for x in xs]
    for r in range(WORLD):
        _copy_loop(recv[r], back, tabs[r].combine)
    for r in range(WORLD):
        assert torch.equal(back[r], xs[r])


def test_balanced_expert_order():
    from primus_turbo_b200.pytorch.dist.expert_parallel import balanced_expert_order, load_imbalance

    g = torch.Generator().manual_seed(0)
    load = torch.softmax(torch.randn(64, generator=g), 0)
    for world in (2, 4, 8):
        order = balanced_expert_order(load, world)
        assert sorted(order.tolist()) == list(range(64))
        for r in range(world):  # each rank's experts are listed in increasing id
            blk = order[r * 64 // world : (r + 1) * 64 // world].tolist()
            assert blk == sorted(blk)
        assert load_imbalance(load[order], world) <= load_imbalance(load, world) + 1e-12
        # the heaviest expert bounds what any placement can reach; its rank still takes E/world experts
        assert load_imbalance(load[order], world) < max(1.1, float(load.max()) * world * 1.1)
    assert balanced_expert_order(torch.zeros(8), 4).tolist() == list(range(8))


def _worker(rank, store_path, seed, out_q, WORLD, E):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    torch.multiprocessing.set_sharing_strategy("file_system")  # handles that any process can open
    store = dist.FileStore(store_path, WORLD)
    dist.init_process_group("gloo", store=store, rank=rank, world_size=WORLD)
    try:
        from primus_turbo_b200.pytorch.dist.expert_parallel import build_peer_plan, expert_parallel_apply_peer
        from primus_turbo_b200.pytorch.dist.peer_exchange import PeerExchange

        regions = {}

        def alloc(nbytes):
            return torch.zeros(nbytes, dtype=torch.uint8).share_memory_()

        def copy(src, dst_ptrs, segs, row_bytes, num_ctas):
            # test stand-in for the device kernel: the exchange hands over raw addresses, so look the
            # shared tensors up by address
            views = [regions[p] for p in dst_ptrs]
            flat = src.contiguous().view(torch.uint8).view(src.shape[0], row_bytes)
            _copy_loop(flat, [v.view(-1, row_bytes) for v in views], segs)

        from multiprocessing.reduction import ForkingPickler
        import pickle

        ex = PeerExchange(None, None, "cpu", capacity_rows=7 * E * WORLD, local_rows=7 * E, copy_fn=copy, alloc_fn=alloc,
                          export_fn=lambda t: bytes(ForkingPickler.dumps(t)), import_fn=pickle.loads)
        orig_region = ex._region

        def region(direction, row_bytes, phase="fwd"):
            out = orig_region(direction, row_bytes, phase)
            for t in out[1]:
                regions[t.data_ptr()] = t
            return out

        ex._region = region
        e_loc = E // WORLD
        results = []
        for step in range(2):  # the second step reuses every region
            counts, xs = _routing(seed, WORLD, E, step)
            x = xs[rank].clone().requires_grad_(True)

            def local_fn(rows, group_lens):
                assert group_lens.tolist() == counts[:, rank * e_loc : (rank + 1) * e_loc].sum(0).tolist()
                outs, start = [], 0
                for i, n in enumerate(group_lens.tolist()):
                    outs.append(_expert_fn(rank * e_loc + i, rows[start : start + n]))
                    start += n
                return torch.cat(outs) if outs else rows

            plan = build_peer_plan(counts[rank], dist.group.WORLD, "cpu")
            assert torch.equal(plan.counts_matrix, counts)
            y = expert_parallel_apply_peer(x, local_fn, ex, plan)
            coeff = torch.arange(y.numel(), dtype=torch.float64).view_as(y) * 1e-2 + 1.0
            (y * coeff).sum().backward()
            results.append((y.detach().tolist(), x.grad.tolist()))
        out_q.put((rank, results))
        dist.barrier()
        ex.close()
    except Exception as exc:  # surface the failure instead of letting the parent wait for a result
        out_q.put((rank, repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("WORLD,E", SHAPES)
def test_peer_exchange_forward_backward_two_steps(WORLD, E):
    seed = 1
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker, args=(r, os.path.join(d, "store"), seed, q, WORLD, E)) for r in range(WORLD)]
        for p in procs:
            p.start()
        results = {}
        for _ in range(WORLD):
            r, res = q.get(timeout=180)
            assert not isinstance(res, str), f"rank {r} failed: {res}"
            results[r] = res
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    for step in range(2):
        counts, xs = _routing(seed, WORLD, E, step)
        for r in range(WORLD):
            x = xs[r].clone().requires_grad_(True)
            outs, start = [], 0
            for e in range(E):
                n = int(counts[r, e])
                outs.append(_expert_fn(e, x[start : start + n]))
                start += n
            y_ref = torch.cat(outs)
            coeff = torch.arange(y_ref.numel(), dtype=torch.float64).view_as(y_ref) * 1e-2 + 1.0
            (y_ref * coeff).sum().backward()
            y, gx = results[r][step]
            assert torch.equal(torch.tensor(y, dtype=torch.float64).reshape(-1, H), y_ref.detach())
            assert torch.equal(torch.tensor(gx, dtype=torch.float64).reshape(-1, H), x.grad)


# ---- the single autograd node that overlaps weight quantisation / wgrad with the exchanges ---------------
def _w(seed, E):
    g = torch.Generator().manual_seed(100 + seed)
    return torch.randn(E, 4, H, generator=g, dtype=torch.float64)


def _worker_overlapped(rank, store_path, seed, out_q, WORLD, E):
    from tests.test_expert_parallel_gloo import _TorchSteps

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    torch.multiprocessing.set_sharing_strategy("file_system")
    dist.init_process_group("gloo", store=dist.FileStore(store_path, WORLD), rank=rank, world_size=WORLD)
    try:
        import pickle
        from multiprocessing.reduction import ForkingPickler

        from primus_turbo_b200.pytorch.dist.expert_parallel import build_peer_plan, ep_grouped_gemm_fp8_peer
        from primus_turbo_b200.pytorch.dist.peer_exchange import PeerExchange

        regions = {}

        def copy(src, dst_ptrs, segs, row_bytes, num_ctas):
            flat = src.contiguous().view(torch.uint8).view(src.shape[0], row_bytes)
            _copy_loop(flat, [regions[p].view(-1, row_bytes) for p in dst_ptrs], segs)

        ex = PeerExchange(None, None, "cpu", capacity_rows=7 * E * WORLD, local_rows=7 * E, copy_fn=copy,
                          alloc_fn=lambda n: torch.zeros(n, dtype=torch.uint8).share_memory_(),
                          export_fn=lambda t: bytes(ForkingPickler.dumps(t)), import_fn=pickle.loads)
        orig_region = ex._region

        def region(direction, row_bytes, phase="fwd"):
            out = orig_region(direction, row_bytes, phase)
            for t in out[1]:
                regions[t.data_ptr()] = t
            return out

        ex._region = region
        counts, xs = _routing(seed, WORLD, E)
        e_loc = E // WORLD
        x = xs[rank].clone().requires_grad_(True)
        w = _w(seed, E)[rank * e_loc : (rank + 1) * e_loc].clone().requires_grad_(True)
        plan = build_peer_plan(counts[rank], dist.group.WORLD, "cpu")
        y = ep_grouped_gemm_fp8_peer(x, w, ex, plan, overlap=True, steps=_TorchSteps())
        coeff = torch.arange(y.numel(), dtype=torch.float64).view_as(y) * 1e-2 + 1.0
        (y * coeff).sum().backward()
        out_q.put((rank, y.detach().tolist(), x.grad.tolist(), w.grad.tolist()))
        dist.barrier()
        ex.close()
    except Exception as exc:
        out_q.put((rank, repr(exc), None, None))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("WORLD,E", SHAPES)
def test_peer_exchange_overlapped_node(WORLD, E):
    from tests.test_expert_parallel_gloo import N_OUT

    seed = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker_overlapped, args=(r, os.path.join(d, "store"), seed, q, WORLD, E)) for r in range(WORLD)]
        for p in procs:
            p.start()
        results = {}
        for _ in range(WORLD):
            r, y, gx, gw = q.get(timeout=180)
            assert gx is not None, f"rank {r} failed: {y}"
            results[r] = (torch.tensor(y, dtype=torch.float64).reshape(-1, N_OUT),
                          torch.tensor(gx, dtype=torch.float64).reshape(-1, H),
                          torch.tensor(gw, dtype=torch.float64).reshape(-1, N_OUT, H))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    counts, xs = _routing(seed, WORLD, E)
    w_full = _w(seed, E).clone().requires_grad_(True)
    x_all, y_all = [], []
    for r in range(WORLD):
        x = xs[r].clone().requires_grad_(True)
        outs, start = [], 0
        for e in range(E):
            n = int(counts[r, e])
            outs.append(x[start : start + n] @ w_full[e].t())
            start += n
        y_ref = torch.cat(outs)
        coeff = torch.arange(y_ref.numel(), dtype=torch.float64).view_as(y_ref) * 1e-2 + 1.0
        x_all.append(x)
        y_all.append((y_ref, coeff))
    sum((y * c).sum() for y, c in y_all).backward()
    e_loc = E // WORLD
    for r in range(WORLD):
        assert torch.allclose(results[r][0], y_all[r][0].detach(), rtol=0, atol=1e-12)
        assert torch.allclose(results[r][1], x_all[r].grad, rtol=0, atol=1e-12)
        assert torch.allclose(results[r][2], w_full.grad[r * e_loc : (r + 1) * e_loc], rtol=0, atol=1e-12)
