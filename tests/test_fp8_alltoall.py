"""``FP8AllToAll`` (primus_turbo/pytorch/dist/fp8_alltoall.py:25-194; reference test
tests/pytorch/dist/test_fp8_alltoall.py).

CPU, gloo, two ranks: the unquantised path (splits, the transposed splits of the backward pass).
GPU, NCCL, two ranks (skipped with fewer GPUs): the FP8 path against the same exchange in bf16, and against
an exact restatement -- each rank's rows quantised tensorwise with that rank's scale, dequantised with the
smallest ``scale_inv`` of the group."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

WORLD = 2
SPLITS = [[3, 5], [4, 2]]  # SPLITS[r][d]: rows rank r sends to rank d
H = 16


def _inputs(rank, dtype=torch.float64):
    g = torch.Generator().manual_seed(7 + rank)
    return torch.randn(sum(SPLITS[rank]), H, generator=g, dtype=torch.float32).to(dtype) * (1.0 + rank)


def _worker(rank, store_path, q, backend, quant):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    if backend == "nccl":
        torch.cuda.set_device(rank)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # a failing rank must not leave NVLink multicast objects behind
    dist.init_process_group(backend, store=dist.FileStore(store_path, WORLD), rank=rank, world_size=WORLD)
    try:
        from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, Format
        from primus_turbo_b200.pytorch.dist import FP8AllToAll

        dev = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
        dtype = torch.bfloat16 if backend == "nccl" else torch.float64
        x = _inputs(rank, dtype).to(dev).requires_grad_(True)
        in_splits = SPLITS[rank]
        out_splits = [SPLITS[s][rank] for s in range(WORLD)]
        cfg = Float8QuantConfig(format=Format.HYBRID)
        y = FP8AllToAll.apply(dist.group.WORLD, x, out_splits, in_splits, quant, quant, cfg)
        go = torch.arange(y.numel(), dtype=torch.float32).view_as(y).to(dev).to(dtype) * 1e-2 + rank
        y.backward(go)
        q.put((rank, y.detach().double().cpu().tolist(), x.grad.double().cpu().tolist(), go.double().cpu().tolist()))
        dist.barrier()
    except Exception as exc:
        q.put((rank, repr(exc), None, None))
        raise
    finally:
        dist.destroy_process_group()


def _run(backend, quant):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker, args=(r, os.path.join(d, "store"), q, backend, quant)) for r in range(WORLD)]
        for p in procs:
            p.start()
        res = {}
        try:
            for _ in range(WORLD):
                r, y, gx, go = q.get(timeout=180)
                assert gx is not None, f"rank {r} failed: {y}"
                res[r] = (torch.tensor(y), torch.tensor(gx), torch.tensor(go))
            for p in procs:
                p.join(timeout=60)
                assert p.exitcode == 0
        finally:
            for p in procs:  # after a failure: end exactly the children started here
                if p.is_alive():
                    p.terminate()
                    p.join(timeout=30)
    return res


def _route(per_rank):
    """what each rank receives when rank s sends per_rank[s] split by SPLITS[s]"""
    out = []
    for d in range(WORLD):
        parts = []
        for s in range(WORLD):
            lo = sum(SPLITS[s][:d])
            parts.append(per_rank[s][lo : lo + SPLITS[s][d]])
        out.append(torch.cat(parts))
    return out


def _route_back(per_rank):
    """transpose of _route: rank d's rows go back to where they came from"""
    out = []
    for s in range(WORLD):
        parts = []
        for d in range(WORLD):
            lo = sum(SPLITS[r][d] for r in range(s))
            parts.append(per_rank[d][lo : lo + SPLITS[s][d]])
        out.append(torch.cat(parts))
    return out


def test_unquantised_exchange_and_its_backward_on_cpu():
    res = _run("gloo", quant=False)
    want = _route([_inputs(r) for r in range(WORLD)])
    back = _route_back([res[r][2] for r in range(WORLD)])
    for r in range(WORLD):
        assert torch.equal(res[r][0], want[r])
        assert torch.equal(res[r][1], back[r])


@pytest.mark.gpu
def test_fp8_exchange_on_two_gpus():
    if torch.cuda.device_count() < WORLD:
        pytest.skip("needs 2 GPUs")
    from oracle import fp8_oracle as O

    res = _run("nccl", quant=True)
    xs = [_inputs(r, torch.bfloat16) for r in range(WORLD)]

    def wire(ts, fp8):
        qs = [O.quant_tensorwise(t, fp8) for t in ts]
        s_min = torch.stack([s for _, s in qs]).min()
        return [(q.float() * s_min).to(torch.bfloat16) for q, _ in qs]

    want = _route(wire(xs, torch.float8_e4m3fn))
    gos = [res[r][2].to(torch.bfloat16) for r in range(WORLD)]
    back = _route_back(wire(gos, torch.float8_e5m2))
    for r in range(WORLD):
        assert torch.equal(res[r][0], want[r].double())
        assert torch.equal(res[r][1], back[r].double())
