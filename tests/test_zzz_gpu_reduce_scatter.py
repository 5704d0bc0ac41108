"""ReduceScatter on the GPU: the two kernels of ``csrc/kernels/scatter.cuh`` through the
service, against a PyTorch fp64 reduction of the same inputs. Ranks are threads of this
process; with one GPU they all sit on device 0 (one cooperative launch carries every rank),
with more GPUs also one rank per device, which adds the in-switch variant.

Collected after every other test file: these kernels are newer than the rest of the suite.
"""
import pytest
import torch

from helpers import fresh_comm_id, run_ranks

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.fixture(scope="module")
def svc(service):
    assert service.backend() == "cuda", "GPU tests must run against the CUDA backend, not a host fallback"
    return service


def _case(M, n, dtype, count, algo, devices, op="sum", in_place=False):
    cid = fresh_comm_id()
    esz = torch.empty((), dtype=dtype).element_size()

    def rank_fn(r):
        dev = devices[r]
        torch.cuda.set_device(dev)
        torch.cuda.set_stream(torch.cuda.Stream(device=dev))   # one stream per rank of a communicator
        a, b = M.Buffer(count * n * esz + 64, dev), M.Buffer(count * esz + 64, dev)
        g = torch.Generator().manual_seed(500 + r)
        x = ((torch.rand(count * n, generator=g) * 2 - 1).to(dtype) if dtype.is_floating_point
             else torch.randint(-1000, 1000, (count * n,), generator=g).to(dtype))
        s = a.tensor(dtype, count * n)
        s.copy_(x)
        d = s[r * count:(r + 1) * count] if in_place else b.tensor(dtype, count)
        c = M.Communicator(cid, r, n, device=dev)
        c.reduce_scatter(s, d, op=op, algo=algo)
        torch.cuda.synchronize(dev)
        got, plan, q = d.cpu(), c.last_plan(), c.query()
        c.destroy()
        return x, got, plan, q

    outs = run_ranks(n, rank_fn)
    xs = torch.stack([o[0].double() for o in outs])
    full = {"sum": xs.sum(0), "max": xs.max(0).values, "avg": xs.sum(0) / n}[op]
    for r, (_, got, plan, q) in enumerate(outs):
        assert q["device_error"] == 0 and q["async_error"] == 0
        if algo != "auto":
            assert plan[0] == algo, f"asked for {algo}, service ran {plan[0]}"
        want = full[r * count:(r + 1) * count]
        if dtype.is_floating_point:
            tol = {torch.float32: 1e-5, torch.float64: 1e-12}.get(dtype, 1.6e-2)
            assert torch.allclose(got.double(), want, rtol=tol, atol=tol * n), f"{algo} {dtype} n={n} count={count}"
        else:
            assert torch.equal(got.to(torch.int64), want.to(torch.int64))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
@pytest.mark.parametrize("n", [2, 4, 8])
def test_reduce_scatter_single_gpu(svc, dtype, n):
    for count in (1, 1000, 4096, 65536 + 3):
        _case(svc, n, dtype, count, "rs_direct", [0] * n)
    _case(svc, n, dtype, 4096, "rs_direct", [0] * n, in_place=True)
    _case(svc, n, dtype, 1000, "auto", [0] * n, op="avg" if dtype.is_floating_point else "max")


def test_reduce_scatter_single_rank(svc):
    _case(svc, 1, torch.float32, 1000, "auto", [0])


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("algo", ["rs_direct", "rs_nvls", "auto"])
def test_reduce_scatter_multi_gpu(svc, algo):
    n = min(_ngpu(), 8)
    for dtype in (torch.float32, torch.bfloat16):
        for count in (4096, 1 << 20):
            _case(svc, n, dtype, count, algo, list(range(n)))
        _case(svc, n, dtype, 1 << 16, algo, list(range(n)), in_place=True)
