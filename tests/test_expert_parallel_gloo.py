"""CPU, world sizes 2 and 4 over gloo: the expert-parallel exchange (count all-gather, row all-to-all,
expert-major permutation and the way back) against a single-process evaluation, forward and
backward, including experts that receive no rows."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

H = 5
# (world size, experts): 3, 2 and 1 experts per rank; with one expert per rank the owner of the unused expert gets no row
SHAPES = [(2, 6), (4, 8), (4, 4)]


def _routing(seed, WORLD, E):
    g = torch.Generator().manual_seed(seed)
    counts = torch.randint(0, 7, (WORLD, E), generator=g)
    counts[:, 1] = 0  # an expert nobody routes to
    if E > 4:
        counts[1, 4] = 0
    xs = [torch.randn(int(counts[r].sum()), H, generator=g, dtype=torch.float64) for r in range(WORLD)]
    return counts, xs


def _expert_fn(e_global: int, rows: torch.Tensor) -> torch.Tensor:
    return rows * (e_global + 1.0) + rows.pow(2) * 0.5


def _worker(rank, store_path, seed, out_q, WORLD, E):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    store = dist.FileStore(store_path, WORLD)
    dist.init_process_group("gloo", store=store, rank=rank, world_size=WORLD)
    try:
        from primus_turbo_b200.pytorch.dist.expert_parallel import build_exchange_plan, expert_parallel_apply

        counts, xs = _routing(seed, WORLD, E)
        x = xs[rank].clone().requires_grad_(True)
        e_loc = E // WORLD

        def local_fn(rows, group_lens):
            assert group_lens.tolist() == counts[:, rank * e_loc : (rank + 1) * e_loc].sum(0).tolist()
            outs, start = [], 0
            for i, n in enumerate(group_lens.tolist()):
                outs.append(_expert_fn(rank * e_loc + i, rows[start : start + n]))
                start += n
            return torch.cat(outs) if outs else rows

        plan = build_exchange_plan(counts[rank])
        assert plan.send_splits == counts[rank].view(WORLD, e_loc).sum(1).tolist()
        # counts already on the host: gathered over a CPU group, same plan
        plan_h = build_exchange_plan(counts[rank], counts_host=counts[rank], host_group=dist.group.WORLD)
        assert plan_h.send_splits == plan.send_splits and plan_h.recv_splits == plan.recv_splits
        assert torch.equal(plan_h.gather_index, plan.gather_index) and torch.equal(plan_h.group_lens, plan.group_lens)
        y = expert_parallel_apply(x, counts[rank], local_fn, plan=plan)
        coeff = torch.arange(y.numel(), dtype=torch.float64).view_as(y) * 1e-2 + 1.0
        (y * coeff).sum().backward()
        out_q.put((rank, y.detach().tolist(), x.grad.tolist()))  # plain lists: no shared-memory handles
        dist.barrier()
    except Exception as exc:  # surface the failure instead of letting the parent wait for a result
        out_q.put((rank, repr(exc), None))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("WORLD,E", SHAPES)
@pytest.mark.parametrize("seed", [0, 1])
def test_expert_parallel_exchange(seed, WORLD, E):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "store")
        procs = [ctx.Process(target=_worker, args=(r, path, seed, q, WORLD, E)) for r in range(WORLD)]
        for p in procs:
            p.start()
        results = {}
        for _ in range(WORLD):
            r, y, gx = q.get(timeout=120)
            assert gx is not None, f"rank {r} failed: {y}"
            results[r] = (torch.tensor(y, dtype=torch.float64).reshape(-1, H), torch.tensor(gx, dtype=torch.float64).reshape(-1, H))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    counts, xs = _routing(seed, WORLD, E)
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
        assert torch.equal(results[r][0], y_ref.detach())
        assert torch.allclose(results[r][1], x.grad, rtol=0, atol=0)


# ---- the overlapped single-node form (one autograd node around both exchanges) -------------------
N_OUT = 4


class _TorchSteps:
    """Plain-torch stand-ins for the device steps: 'quantised' tensors are the tensors themselves."""

    def offsets(self, lens):
        return torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(lens, 0)])

    def quant_weight(self, w):
        return w, torch.ones(())

    def quant_rows(self, x, lens, offs, fwd):
        return x, x, None, None, lens, offs

    @staticmethod
    def _per_group(offs, fn):
        o = offs.tolist()
        return [fn(g, o[g], o[g + 1]) for g in range(len(o) - 1)]

    def fwd(self, a_row, a_s_row, b8, b_s, lens, offs):
        return torch.cat(self._per_group(offs, lambda g, lo, hi: a_row[lo:hi] @ b8[g].t()))

    def dgrad(self, g_row, g_s_row, b8, b_s, lens, offs):
        return torch.cat(self._per_group(offs, lambda g, lo, hi: g_row[lo:hi] @ b8[g]))

    def wgrad(self, a_col, a_s_col, g_col, g_s_col, vk_lens, vk_offs, num_cu=None):
        return torch.stack(self._per_group(vk_offs, lambda g, lo, hi: g_col[lo:hi].t() @ a_col[lo:hi]))


def _weights(seed, E):
    g = torch.Generator().manual_seed(100 + seed)
    return torch.randn(E, N_OUT, H, generator=g, dtype=torch.float64)


def _worker_overlapped(rank, store_path, seed, out_q, WORLD, E):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    store = dist.FileStore(store_path, WORLD)
    dist.init_process_group("gloo", store=store, rank=rank, world_size=WORLD)
    try:
        from primus_turbo_b200.pytorch.dist.expert_parallel import ep_grouped_gemm_fp8

        counts, xs = _routing(seed, WORLD, E)
        e_loc = E // WORLD
        x = xs[rank].clone().requires_grad_(True)
        w = _weights(seed, E)[rank * e_loc : (rank + 1) * e_loc].clone().requires_grad_(True)
        y = ep_grouped_gemm_fp8(x, w, counts[rank], overlap=True, steps=_TorchSteps())
        coeff = torch.arange(y.numel(), dtype=torch.float64).view_as(y) * 1e-2 + 1.0
        (y * coeff).sum().backward()
        out_q.put((rank, y.detach().tolist(), x.grad.tolist(), w.grad.tolist()))
        dist.barrier()
    except Exception as exc:
        out_q.put((rank, repr(exc), None, None))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("WORLD,E", SHAPES)
@pytest.mark.parametrize("seed", [0, 1])
def test_expert_parallel_overlapped(seed, WORLD, E):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "store")
        procs = [ctx.Process(target=_worker_overlapped, args=(r, path, seed, q, WORLD, E)) for r in range(WORLD)]
        for p in procs:
            p.start()
        results = {}
        for _ in range(WORLD):
            r, y, gx, gw = q.get(timeout=120)
            assert gx is not None, f"rank {r} failed: {y}"
            results[r] = (torch.tensor(y, dtype=torch.float64).reshape(-1, N_OUT),
                          torch.tensor(gx, dtype=torch.float64).reshape(-1, H),
                          torch.tensor(gw, dtype=torch.float64).reshape(-1, N_OUT, H))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    counts, xs = _routing(seed, WORLD, E)
    w_full = _weights(seed, E).clone().requires_grad_(True)
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


# ---- shared-memory gather of the routing counts (ranks on one machine) ---------------------------
def _worker_board(rank, store_path, out_q, WORLD, E):
    import random
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    dist.init_process_group("gloo", store=dist.FileStore(store_path, WORLD), rank=rank, world_size=WORLD)
    try:
        from primus_turbo_b200.pytorch.dist.expert_parallel import SharedCountsBoard, build_exchange_plan

        board = SharedCountsBoard(E)
        rng = random.Random(rank)
        ok = True
        for call in range(40):
            g = torch.Generator().manual_seed(1000 * call)  # every rank can rebuild the whole matrix
            matrix = torch.randint(0, 50, (WORLD, E), generator=g)
            if rng.random() < 0.3:
                time.sleep(rng.random() * 0.003)  # ranks arrive at different times
            got = board.all_gather_counts(matrix[rank])
            ok = ok and torch.equal(got, matrix)
        # the plan built through the board equals the one built through the gloo group
        counts, _ = _routing(0, WORLD, E)
        p_board = build_exchange_plan(counts[rank], counts_host=counts[rank], host_group=board)
        p_gloo = build_exchange_plan(counts[rank], counts_host=counts[rank], host_group=dist.group.WORLD)
        ok = ok and p_board.send_splits == p_gloo.send_splits and p_board.recv_splits == p_gloo.recv_splits
        ok = ok and torch.equal(p_board.gather_index, p_gloo.gather_index)
        ok = ok and torch.equal(p_board.scatter_index, p_gloo.scatter_index)
        ok = ok and torch.equal(p_board.group_lens, p_gloo.group_lens)
        ok = ok and torch.equal(p_board.counts_matrix, p_gloo.counts_matrix)
        dist.barrier()
        board.close()
        out_q.put((rank, bool(ok)))
    except Exception as exc:
        out_q.put((rank, repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("WORLD,E", [(4, 8)])
def test_shared_counts_board(WORLD, E):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker_board, args=(r, os.path.join(d, "store"), q, WORLD, E)) for r in range(WORLD)]
        for p in procs:
            p.start()
        for _ in range(WORLD):
            r, ok = q.get(timeout=180)
            assert ok is True, f"rank {r}: {ok}"
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
