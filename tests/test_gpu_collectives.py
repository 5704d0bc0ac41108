"""GPU tests of the sm_100a kernels through the whole service path. With one GPU
every rank of a communicator sits on cuda:0 and the daemon runs the collective as
one cooperative launch over all ranks' data (kernels that wait on one another must
not be separate launches on one GPU); with two or more GPUs the same tests also run
with one rank per device, which adds the peer-memory and NVLS variants. Every
result is compared with a plain PyTorch fp32/fp64 reduction of the same inputs."""
import ctypes
import os

import pytest
import torch

from helpers import fresh_comm_id, run_ranks

pytestmark = pytest.mark.gpu

AR_ALGOS = ["ar_oneshot", "ar_twoshot", "ar_ring"]
AG_ALGOS = ["ag_pull", "ag_push", "ag_ring"]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.fixture(scope="module")
def svc(service):
    assert service.backend() == "cuda", "GPU tests must run against the CUDA backend, not a host fallback"
    return service


def _own_stream(dev):
    """Each rank thread works on a stream of its own. With stream-memory-operation
    synchronisation a collective call queues "wait until done" on the caller's stream
    right away, so two ranks of one communicator must not share a stream (the second
    rank's "submitted" mark would queue behind the first rank's wait)."""
    torch.cuda.set_device(dev)
    torch.cuda.set_stream(torch.cuda.Stream(device=dev))


def _make(dtype, count, seed):
    g = torch.Generator().manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(count, generator=g) * 2 - 1).to(dtype)
    return torch.randint(-1000, 1000, (count,), generator=g).to(dtype)


def _allreduce_case(M, n, dtype, count, algo, devices, op="sum", in_place=False, offset=0, scale=1.0):
    cid = fresh_comm_id()
    esz = torch.empty((), dtype=dtype).element_size()

    def rank_fn(r):
        dev = devices[r]
        _own_stream(dev)
        nbytes = (count + offset) * esz + 64
        a, b = M.Buffer(nbytes, dev), M.Buffer(nbytes, dev)
        x = _make(dtype, count, 100 + r)
        if op == "prod":
            x = (x.float().abs() * 0.5 + 0.75).to(dtype) if dtype.is_floating_point else (x % 3 + 1)
        s = a.tensor(dtype, count + offset)[offset:]
        d = s if in_place else b.tensor(dtype, count + offset)[offset:]
        s.copy_(x)
        c = M.Communicator(cid, r, n, device=dev)
        c.all_reduce(s, d, op=op, algo=algo, scale=scale)
        torch.cuda.synchronize(dev)
        got = d.cpu()
        plan = c.last_plan()
        q = c.query()
        c.destroy()
        return x, got, plan, q

    outs = run_ranks(n, rank_fn)
    xs = torch.stack([o[0].double() for o in outs])
    if op == "sum":
        want = xs.sum(0)
    elif op == "prod":
        want = xs.prod(0)
    elif op == "max":
        want = xs.max(0).values
    elif op == "min":
        want = xs.min(0).values
    elif op == "avg":
        want = xs.sum(0) / n
    else:
        want = (xs * scale).sum(0)
    for _, got, plan, q in outs:
        assert q["device_error"] == 0 and q["async_error"] == 0
        if algo != "auto":
            assert plan[0] == algo, f"asked for {algo}, service ran {plan[0]}"
        if dtype.is_floating_point:
            tol = {torch.float32: 1e-5, torch.float64: 1e-12}.get(dtype, 1.6e-2)
            assert torch.allclose(got.double(), want, rtol=tol, atol=tol * n), f"{algo} {dtype} n={n} count={count}"
        else:
            assert torch.equal(got.to(torch.int64), want.to(torch.int64))
    # every rank must hold bit-identical results
    for o in outs[1:]:
        assert torch.equal(o[1], outs[0][1])


@pytest.mark.parametrize("algo", AR_ALGOS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32])
@pytest.mark.parametrize("n", [2, 4, 8])
def test_allreduce_single_gpu(svc, algo, dtype, n):
    for count in (1, 1000, 65536 + 3, 1 << 20):
        _allreduce_case(svc, n, dtype, count, algo, [0] * n)


@pytest.mark.parametrize("algo", ["ar_twoshot", "ar_ring"])
def test_allreduce_in_place_and_unaligned(svc, algo):
    _allreduce_case(svc, 4, torch.float32, 50000, algo, [0] * 4, in_place=True)
    _allreduce_case(svc, 4, torch.bfloat16, 50001, algo, [0] * 4, offset=3)      # 6-byte offset: scalar path
    _allreduce_case(svc, 2, torch.float32, 4099, algo, [0] * 2, offset=1, in_place=True)


@pytest.mark.parametrize("op", ["prod", "max", "min", "avg", "premulsum"])
def test_allreduce_ops(svc, op):
    for algo in AR_ALGOS:
        _allreduce_case(svc, 4, torch.float32, 30000, algo, [0] * 4, op=op, scale=0.25)
    _allreduce_case(svc, 2, torch.bfloat16, 30000, "ar_twoshot", [0] * 2, op=op, scale=0.25)


@pytest.mark.parametrize("dtype", [torch.float64, torch.int64, torch.int8, torch.uint8])
def test_allreduce_other_types(svc, dtype):
    _allreduce_case(svc, 2, dtype, 10007, "ar_twoshot", [0, 0]) if dtype not in (torch.int8, torch.uint8) else None
    _allreduce_case(svc, 4, dtype, 4096, "ar_oneshot", [0] * 4, op="max")


def _allgather_case(M, n, nbytes, algo, devices, in_place):
    cid = fresh_comm_id()

    def rank_fn(r):
        dev = devices[r]
        _own_stream(dev)
        out = M.Buffer(nbytes * n + 64, dev)
        full = out.tensor(torch.uint8, nbytes * n)
        full.zero_()
        g = torch.Generator().manual_seed(7 + r)
        x = torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8)
        if in_place:
            mine = full[r * nbytes:(r + 1) * nbytes]
        else:
            src = M.Buffer(nbytes + 64, dev)
            mine = src.tensor(torch.uint8, nbytes)
        mine.copy_(x)
        c = M.Communicator(cid, r, n, device=dev)
        c.all_gather(mine, full, algo=algo)
        torch.cuda.synchronize(dev)
        got = full.cpu()
        plan = c.last_plan()
        q = c.query()
        c.destroy()
        return x, got, plan, q

    outs = run_ranks(n, rank_fn)
    want = torch.cat([o[0] for o in outs])
    for _, got, plan, q in outs:
        assert q["device_error"] == 0
        if algo != "auto":
            assert plan[0] == algo
        assert torch.equal(got, want), f"{algo} n={n} bytes={nbytes} in_place={in_place}"


@pytest.mark.parametrize("algo", AG_ALGOS)
@pytest.mark.parametrize("n", [2, 4, 8])
def test_allgather_single_gpu(svc, algo, n):
    for nbytes in (16, 4096, 1 << 20, 100003):     # the last one is not a multiple of 16: byte path
        _allgather_case(svc, n, nbytes, algo, [0] * n, in_place=False)
    _allgather_case(svc, n, 65536, algo, [0] * n, in_place=True)


def test_single_rank_copy(svc):
    _allreduce_case(svc, 1, torch.float32, 100001, "auto", [0])
    _allgather_case(svc, 1, 5000, "auto", [0], in_place=False)


def test_ring_many_loops_and_reorder(svc):
    """A message much larger than one FIFO round (several loops per channel), then the
    same communicator after a live ring re-order: results must not change."""
    M = svc
    n, count, cid = 4, (24 << 20) // 4, fresh_comm_id()
    port = M.daemon.embedded_admin_port()
    import threading
    sync = threading.Barrier(n)

    def rank_fn(r):
        _own_stream(0)
        a = M.Buffer(count * 4, 0)
        b = M.Buffer(count * 4, 0)
        x = _make(torch.float32, count, 300 + r)
        s, d = a.tensor(torch.float32, count), b.tensor(torch.float32, count)
        s.copy_(x)
        c = M.Communicator(cid, r, n, device=0)
        c.all_reduce(s, d, algo="ar_ring")
        torch.cuda.synchronize()
        first = d.cpu()
        sync.wait()
        if r == 0:
            rep = M.reconfigure(port, [{"communicator_id": cid, "channels": [
                {"channel_id": 0, "ring": [3, 1, 0, 2]}, {"channel_id": 1, "ring": [0, 2, 1, 3]},
                {"channel_id": 2, "ring": [2, 3, 0, 1]}]}])
            assert rep["status"] == "ok", rep
        sync.wait()
        d.zero_()
        c.all_reduce(s, d, algo="ar_ring")
        torch.cuda.synchronize()
        second = d.cpu()
        q = c.query()
        plan = c.last_plan()
        sync.wait()
        c.destroy()
        return x, first, second, q, plan

    outs = run_ranks(n, rank_fn, timeout=300)
    want = torch.stack([o[0].double() for o in outs]).sum(0)
    for _, first, second, q, plan in outs:
        assert torch.allclose(first.double(), want, rtol=1e-5, atol=1e-5)
        assert torch.allclose(second.double(), want, rtol=1e-5, atol=1e-5)
        assert q["config_epoch"] == 1 and plan == ("ar_ring", 3)


def test_bounded_wait_reports_instead_of_hanging(svc):
    """A kernel whose peer never shows up gives up after its bound, reports a
    start-barrier timeout through the status block, and the context stays usable."""
    from mccs_b200 import _lib
    lib = _lib.daemon_lib()
    lib.mccs_selftest_bounded_wait.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_uint),
                                               ctypes.POINTER(ctypes.c_double)]
    lib.mccs_selftest_bounded_wait.restype = ctypes.c_int
    err, ms = ctypes.c_uint(0), ctypes.c_double(0)
    rc = lib.mccs_selftest_bounded_wait(0, 300, ctypes.byref(err), ctypes.byref(ms))
    assert rc == 0
    assert err.value == 1            # kDevTimeoutStart
    assert 250 <= ms.value < 3000
    # still healthy afterwards
    _allreduce_case(svc, 2, torch.float32, 1000, "ar_twoshot", [0, 0])


# ---------------------------------------------------------------------------------------------
# two or more GPUs: one rank per device, peer memory and NVLS
# ---------------------------------------------------------------------------------------------
multi = pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")


@multi
@pytest.mark.parametrize("algo", AR_ALGOS + ["ar_nvls_oneshot", "ar_nvls_twoshot", "auto"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_allreduce_multi_gpu(svc, algo, dtype):
    n = min(_ngpu(), 8)
    nvls = "nvls=on" in svc.daemon.describe_embedded()
    if "nvls" in algo and not nvls:
        pytest.skip("this box has no NVLS multicast")
    for count in (1000, 65536 + 8, 4 << 20):
        _allreduce_case(svc, n, dtype, count, algo, list(range(n)))
    if algo in ("ar_twoshot", "ar_nvls_twoshot", "ar_ring"):
        _allreduce_case(svc, n, dtype, 1 << 20, algo, list(range(n)), in_place=True)


@multi
@pytest.mark.parametrize("algo", AG_ALGOS + ["ag_nvls", "auto"])
def test_allgather_multi_gpu(svc, algo):
    n = min(_ngpu(), 8)
    nvls = "nvls=on" in svc.daemon.describe_embedded()
    if "nvls" in algo and not nvls:
        pytest.skip("this box has no NVLS multicast")
    for nbytes in (4096, 1 << 20, 8 << 20):
        _allgather_case(svc, n, nbytes, algo, list(range(n)), in_place=False)
    _allgather_case(svc, n, 1 << 20, algo, list(range(n)), in_place=True)


@multi
@pytest.mark.parametrize("algo", ["ar_nvls_twoshot", "ar_twoshot", "ag_nvls", "ag_push"])
def test_back_to_back_on_poisoned_buffers_multi_gpu(svc, algo):
    """200 collectives back to back on each rank's stream with no host synchronisation in
    between: before every call the output is poisoned (NaN / 0xFF) and the input changes, after
    every call a kernel on the same stream counts the elements that differ from what that
    iteration must produce. This is the ordering stress for the kernels whose last remote
    stores are followed only by the closing barrier's flag (multimem.st, then a unicast
    release store): a store that could still be in flight when the peer passes the barrier
    shows up as a poisoned or stale element in some iteration."""
    n = min(_ngpu(), 8)
    nvls = "nvls=on" in svc.daemon.describe_embedded()
    if "nvls" in algo and not nvls:
        pytest.skip("this box has no NVLS multicast")
    cid = fresh_comm_id()
    is_ar = algo.startswith("ar_")
    count = 300000            # fp32 elements (AllReduce) / bytes per rank (AllGather): 16-byte multiples, several CTAs

    def rank_fn(r):
        _own_stream(r)
        if is_ar:
            a, b = svc.Buffer(count * 4, r), svc.Buffer(count * 4, r)
            s, d = a.tensor(torch.float32, count), b.tensor(torch.float32, count)
        else:
            a, b = svc.Buffer(count, r), svc.Buffer(count * n, r)
            s, d = a.tensor(torch.uint8, count), b.tensor(torch.uint8, count * n)
        comm = svc.Communicator(cid, r, n, device=r)
        bad = torch.zeros((), dtype=torch.int64, device=f"cuda:{r}")
        for it in range(200):
            if is_ar:
                s.fill_(float(r + 1) + 0.25 * it)
                d.fill_(float("nan"))
                comm.all_reduce(s, d, algo=algo)
                want = float(n * (n + 1) // 2) + 0.25 * it * n
                bad += (d != want).sum()
            else:
                s.fill_((r * 31 + it) % 251)
                d.fill_(255)
                comm.all_gather(s, d, algo=algo)
                for q in range(n):
                    bad += (d[q * count:(q + 1) * count] != (q * 31 + it) % 251).sum()
        torch.cuda.synchronize()
        q = comm.query()
        comm.destroy()
        return int(bad.item()), q["async_error"], q["device_error"]

    for bad, async_error, device_error in run_ranks(n, rank_fn, timeout=300.0):
        assert bad == 0 and async_error == 0 and device_error == 0
