"""End-to-end tests of the service on the host backend (no GPU): client shim ->
control socket -> daemon -> per-device proxies -> rendezvous -> planner -> QoS
admission -> CPU collectives. Ranks are threads of the test process; every rank
owns a communicator handle and its own request/completion rings, like separate
applications would."""
import torch
import pytest

from helpers import fresh_comm_id, run_ranks

FLOAT_TYPES = [torch.float32, torch.float64, torch.float16, torch.bfloat16]
INT_TYPES = [torch.int32, torch.int64, torch.int8, torch.uint8]


def _make(dtype, count, seed):
    g = torch.Generator().manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(count, generator=g) * 2 - 1).to(dtype)
    hi = 5 if dtype in (torch.int8, torch.uint8) else 1000
    lo = 0 if dtype == torch.uint8 else -hi
    return torch.randint(lo, hi, (count,), generator=g).to(dtype)


@pytest.mark.parametrize("nranks", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", FLOAT_TYPES + INT_TYPES)
def test_allreduce_sum(service, nranks, dtype):
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    cid, count = fresh_comm_id(), 3001

    def rank_fn(r):
        buf, out = M.Buffer(count * 8, r), M.Buffer(count * 8, r)
        x = _make(dtype, count, r)
        s, d = buf.tensor(dtype, count), out.tensor(dtype, count)
        s.copy_(x)
        c = M.Communicator(cid, r, nranks, device=r)
        c.all_reduce(s, d)
        res = d.clone()
        c.all_reduce(s)   # in place
        inplace = s.clone()
        c.destroy()
        return x, res, inplace

    outs = run_ranks(nranks, rank_fn)
    if dtype.is_floating_point:
        want = sum(o[0].double() for o in outs)
        tol = {torch.float32: 1e-5, torch.float64: 1e-12}.get(dtype, 2e-2)
        for _, res, inplace in outs:
            assert torch.allclose(res.double(), want, rtol=tol, atol=tol * nranks)
            assert torch.equal(res, inplace)
    else:
        want = sum(o[0].to(torch.int64) for o in outs).to(dtype)
        for _, res, inplace in outs:
            assert torch.equal(res, want)
            assert torch.equal(inplace, want)


@pytest.mark.parametrize("op", ["prod", "max", "min", "avg", "premulsum"])
def test_allreduce_ops(service, op):
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    n, count, cid = 4, 777, fresh_comm_id()

    def rank_fn(r):
        buf = M.Buffer(count * 4, r)
        x = _make(torch.float32, count, 10 + r) + 1.5
        s = buf.tensor(torch.float32, count)
        s.copy_(x)
        c = M.Communicator(cid, r, n, device=r)
        c.all_reduce(s, op=op, scale=0.5)
        c.destroy()
        return x, s.clone()

    outs = run_ranks(n, rank_fn)
    xs = torch.stack([o[0] for o in outs])
    want = {"prod": xs.prod(0), "max": xs.max(0).values, "min": xs.min(0).values, "avg": xs.sum(0) / n,
            "premulsum": (xs * 0.5).sum(0)}[op]
    for _, got in outs:
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("nranks", [2, 3, 8])
def test_allgather(service, nranks):
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    cid, per = fresh_comm_id(), 1000

    def rank_fn(r):
        out = M.Buffer(per * 4 * nranks, r)
        full = out.tensor(torch.float32, per * nranks)
        full.zero_()
        mine = full[r * per:(r + 1) * per]
        mine.copy_(torch.arange(per, dtype=torch.float32) + r * 1e6)   # rank * 1e6 + index: every element names its origin
        c = M.Communicator(cid, r, nranks, device=r)
        c.all_gather(mine, full)        # in place: send = recv + rank*bytes
        c.destroy()
        return full.clone()

    outs = run_ranks(nranks, rank_fn)
    want = torch.cat([torch.arange(per, dtype=torch.float32) + r * 1e6 for r in range(nranks)])
    for got in outs:
        assert torch.equal(got, want)


def test_config1_two_rank_reference_shapes(service):
    """The smallest end-to-end configuration: 2 ranks, AllReduce sum fp32 count=262144 of N(0,1)
    (seed 0) and AllGather fp32 of 65536 per rank with rank*1e6+index."""
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    cid = fresh_comm_id()
    g = torch.Generator().manual_seed(0)
    data = [torch.randn(262144, generator=g) for _ in range(2)]

    def rank_fn(r):
        a, b = M.Buffer(262144 * 4, r), M.Buffer(65536 * 4 * 2, r)
        s = a.tensor(torch.float32, 262144)
        s.copy_(data[r])
        c = M.Communicator(cid, r, 2, device=r)
        c.all_reduce(s, algo="ar_ring")
        full = b.tensor(torch.float32, 65536 * 2)
        full[r * 65536:(r + 1) * 65536] = torch.arange(65536, dtype=torch.float32) + r * 1e6
        c.all_gather(full[r * 65536:(r + 1) * 65536], full, algo="ag_ring")
        plan = c.last_plan()
        c.destroy()
        return s.clone(), full.clone(), plan

    outs = run_ranks(2, rank_fn)
    want = (data[0].double() + data[1].double()).float()
    for s, full, plan in outs:
        assert torch.allclose(s, want, rtol=1e-5, atol=1e-6)
        assert torch.equal(full, torch.cat([torch.arange(65536, dtype=torch.float32) + r * 1e6 for r in range(2)]))
        assert plan[0] == "ag_ring"


def test_back_to_back_and_group(service):
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    n, cid, count = 4, fresh_comm_id(), 512
    import threading
    done = threading.Barrier(n)

    def rank_fn(r):
        bufs = [M.Buffer(count * 4, r) for _ in range(16)]
        ts = [b.tensor(torch.float32, count) for b in bufs]
        for i, t in enumerate(ts):
            t.fill_(float(r + i))
        c = M.Communicator(cid, r, n, device=r)
        with M.group():                       # 16 back-to-back all-reduces, one completion wait
            for t in ts:
                c.all_reduce(t)
        for _ in range(200):                  # more than the ring depth and the slot count
            c.all_reduce(ts[0])
        q = c.query()
        done.wait()     # a communicator whose peers have left reports that as an error
        c.destroy()
        return [t.clone() for t in ts], q

    outs = run_ranks(n, rank_fn)
    for ts, q in outs:
        for i in range(1, 16):
            assert torch.all(ts[i] == sum(r + i for r in range(n)))
        assert q["launched"] == 216 and q["async_error"] == 0


def test_mismatch_is_an_error_not_a_hang(service):
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    cid = fresh_comm_id()

    def rank_fn(r):
        buf = M.Buffer(4096, r)
        t = buf.tensor(torch.float32, 1024)
        c = M.Communicator(cid, r, 2, device=r)
        try:
            c.all_reduce(t, count=1024 if r == 0 else 512)
            return None
        except M.client._lib.MccsError as e:
            return e.code
        finally:
            c.destroy()

    codes = run_ranks(2, rank_fn)
    assert codes == [-8, -8]      # mccsMismatch on both ranks


def test_ranks_must_agree_on_the_scale_factor(service):
    """PreMulSum's multiplier is one per collective (every source gets the same factor): ranks
    that pass different factors get mccsMismatch instead of rank 0's factor silently."""
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    cid = fresh_comm_id()

    def rank_fn(r):
        buf = M.Buffer(4096, r)
        t = buf.tensor(torch.float32, 1024)
        t.fill_(1.0)
        c = M.Communicator(cid, r, 2, device=r)
        try:
            c.all_reduce(t, op="premulsum", scale=0.5)
            agreed = float(t[0])
            c2 = None
        except M.client._lib.MccsError as e:
            c.destroy()
            return ("first", e.code)
        try:
            c.all_reduce(t, op="premulsum", scale=0.5 if r == 0 else 0.25)
            return ("none", agreed)
        except M.client._lib.MccsError as e:
            return (agreed, e.code)
        finally:
            c.destroy()

    assert run_ranks(2, rank_fn) == [(1.0, -8), (1.0, -8)]


def test_buffer_must_come_from_the_service(service):
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    c = M.Communicator(fresh_comm_id(), 0, 1, device=0)
    t = torch.zeros(16)
    with pytest.raises(M.client._lib.MccsError):
        c.all_reduce(t)
    c.destroy()


def test_functional_ops_over_a_communicator(service):
    """`mccs_b200.ops`: the collectives as plain functions, every variant described."""
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    from mccs_b200 import ops
    assert set(ops.VARIANTS) == set(M.client.ALGOS)
    n, cid = 3, fresh_comm_id()

    def rank_fn(r):
        a, b, d = M.Buffer(4096, r), M.Buffer(4096, r), M.Buffer(4096, r)
        x = a.tensor(torch.float32, 1000)
        x.fill_(float(r + 1))
        c = M.Communicator(cid, r, n, device=r)
        y = ops.all_reduce(c, x, b.tensor(torch.float32, 1000), algo="ar_twoshot")
        z = ops.all_reduce(c, x, op="max")                       # in place: returns the input tensor
        assert z is x
        g = ops.all_gather(c, x[:16], d.tensor(torch.float32, 16 * n), algo="ag_pull")
        x[:3 * n] = torch.arange(3 * n).float() + r
        rs = ops.reduce_scatter(c, x[:3 * n], b.tensor(torch.float32, 3, offset_bytes=4000), op="avg")
        assert torch.allclose(rs, torch.arange(3 * n).float()[3 * r:3 * r + 3] + 1.0)    # mean of r over 3 ranks = 1
        x[:3 * n] = 3.0
        out = (y.clone(), x.clone(), g.clone())
        # ordinary tensors are staged through the communicator's arena, which grows on demand
        small = torch.full((1000,), float(r))
        ops.all_reduce(c, small)
        first_arena = ops.arena(c).buffer.nbytes
        big = torch.full((700000,), float(r + 1))
        ops.all_reduce(c, big, op="avg")
        assert ops.arena(c).buffer.nbytes > first_arena
        assert torch.all(small == 3.0) and torch.all(big == 2.0)
        flags = torch.tensor([r == 0, True, False])               # an element type the kernels do not have: staged as fp32
        ops.all_reduce(c, flags, op="max")
        assert flags.tolist() == [True, True, False]
        ops.arena(c).release()
        c.destroy()
        return out

    for y, x, g in run_ranks(n, rank_fn):
        assert torch.all(y == 6.0) and torch.all(x == 3.0) and torch.all(g == 3.0)
    with pytest.raises(ValueError):
        ops.local_all_reduce_no_alloc([torch.zeros(8)])          # CPU tensors are refused, not silently summed


def test_an_id_can_be_taken_again_while_peers_still_let_go(service):
    """A rank that destroys its communicator and creates the next one under the same id is
    only ahead of its peers: the request waits until the old communicator is gone. An id held
    by an intact communicator is refused at once."""
    import time
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    cid = fresh_comm_id()

    def rank_fn(r):
        buf = M.Buffer(4096, r)
        t = buf.tensor(torch.float32, 256)
        c = M.Communicator(cid, r, 2, device=r)
        t.fill_(float(r + 1))
        c.all_reduce(t)
        first = float(t[0])
        refused, took = None, 0.0
        if r == 0:
            t0 = time.time()
            try:
                M.Communicator(cid, 0, 2, device=0)       # nobody has left: the id is simply in use
            except Exception as e:
                refused = getattr(e, "code", None)
            took = time.time() - t0
        else:
            time.sleep(0.5)       # rank 0 is back for the id long before rank 1 lets go of it
        c.destroy()
        c = M.Communicator(cid, r, 2, device=r)
        t.fill_(float(r + 3))
        c.all_reduce(t)
        second = float(t[0])
        c.destroy()
        return first, second, refused, took

    outs = run_ranks(2, rank_fn)
    assert [o[0] for o in outs] == [3.0, 3.0] and [o[1] for o in outs] == [7.0, 7.0]
    assert outs[0][2] == -1 and outs[0][3] < 1.0


def test_collectives_refuse_cuda_graph_capture(service, monkeypatch):
    """Every collective asks the daemon for its barrier epoch and ticket when it is called, so
    one that was captured into a CUDA graph would replay stale values: the call is refused
    (checked here with a stand-in for torch's capture query; the check itself only runs for
    CUDA communicators)."""
    from mccs_b200 import client
    M = service
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: True)
    with pytest.raises(M.MccsError) as e:
        client._refuse_capture()
    assert getattr(e.value, "code", None) == -9
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    client._refuse_capture()          # not capturing: nothing happens

    def broken():
        raise RuntimeError("no CUDA runtime")
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", broken)
    client._refuse_capture()          # the query itself fails: treated as not capturing
    # a host communicator never asks
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: True)
    if M.backend() == "host":
        cid = fresh_comm_id()
        buf = M.Buffer(64, 0)
        c = M.Communicator(cid, 0, 1, device=0)
        c.all_reduce(buf.tensor(torch.float32, 16))
        c.destroy()
