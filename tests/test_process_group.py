"""The torch.distributed backend and the data-parallel driver, as separate client
processes of a stand-alone ``mccsd`` (host backend): the full IPC path — control
socket, fd passing for allocations and the request/completion rings."""
import os
import socket
import subprocess
import sys
import tempfile

import pytest

from helpers import REPO, write_config

WORKER = r"""
import os, sys, torch, torch.distributed as dist
import mccs_b200.process_group as mpg
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"])
dist.init_process_group("mccs", init_method=f"tcp://127.0.0.1:{os.environ['PORT']}", rank=rank, world_size=n)
t = torch.arange(10, dtype=torch.float32) + rank
dist.all_reduce(t)
assert torch.equal(t, sum(torch.arange(10, dtype=torch.float32) + r for r in range(n))), t
h = (torch.arange(7) + rank).to(torch.bfloat16); dist.all_reduce(h, op=dist.ReduceOp.AVG)
assert torch.allclose(h.float(), torch.arange(7).float() + (n - 1) / 2, atol=0.1)
b = torch.full((5,), float(rank)); dist.broadcast(b, src=1); assert torch.all(b == 1)
# bit-exact for every dtype and odd sizes: negative zero, NaN, bool, 3-byte tails, strided views
nz = torch.tensor([-0.0, float("nan"), float("-inf"), 1.5]) if rank == 0 else torch.ones(4)
dist.broadcast(nz, src=0); assert nz.view(torch.int32).tolist() == torch.tensor([-0.0, float("nan"), float("-inf"), 1.5]).view(torch.int32).tolist()
bb = torch.tensor([True, False, True]) if rank == 1 else torch.zeros(3, dtype=torch.bool)
dist.broadcast(bb, src=1); assert bb.tolist() == [True, False, True]
h = (torch.arange(7, dtype=torch.float16) - 3) if rank == 0 else torch.zeros(7, dtype=torch.float16)
dist.broadcast(h, src=0); assert h.tolist() == (torch.arange(7, dtype=torch.float16) - 3).tolist()
sv = torch.zeros(4, 6); col = sv[:, 1:4]
if rank == 1: col.copy_(torch.arange(12.).reshape(4, 3))
dist.broadcast(col, src=1); assert torch.equal(sv[:, 1:4], torch.arange(12.).reshape(4, 3)) and float(sv[:, 0].abs().sum()) == 0
outs = [torch.empty(3, dtype=torch.int64) for _ in range(n)]
dist.all_gather(outs, torch.full((3,), rank, dtype=torch.int64))
assert all(torch.all(o == r) for r, o in enumerate(outs))
big = torch.empty(n * 4); dist.all_gather_into_tensor(big, torch.full((4,), float(rank)))
assert torch.equal(big, torch.arange(n).repeat_interleave(4).float())
m = torch.tensor([float(rank)]); dist.all_reduce(m, op=dist.ReduceOp.MAX); assert m.item() == n - 1
rs = torch.empty(2); dist.reduce_scatter_tensor(rs, torch.arange(2 * n).float())
assert torch.equal(rs, torch.arange(2 * n).float().reshape(n, 2)[rank] * n)
ro = torch.empty(3, dtype=torch.float16)
dist.reduce_scatter(ro, [torch.full((3,), float(rank + q), dtype=torch.float16) for q in range(n)], op=dist.ReduceOp.AVG)
assert torch.allclose(ro.float(), torch.full((3,), sum(r + rank for r in range(n)) / n))
# both tensors in service memory: the service's reduce-scatter runs on them directly
zf, keep_f = mpg.empty(8 * n, torch.float32, device=rank); zo, keep_o = mpg.empty(8, torch.float32, device=rank)
zf.copy_(torch.arange(8 * n).float() + rank); dist.reduce_scatter_tensor(zo, zf)
assert torch.equal(zo, (torch.arange(8 * n).float().reshape(n, 8)[rank]) * n + sum(range(n)))
# a tensor in service memory is reduced in place, without staging
z, keep = mpg.empty(1000, torch.float32, device=rank)
z.fill_(rank + 1.0); assert mpg.in_service_memory(z)
dist.all_reduce(z); assert torch.all(z == n * (n + 1) / 2)
# rooted and personalised collectives, composed from the three the service has
rd = torch.full((6,), float(rank + 1)); dist.reduce(rd, dst=1)
assert torch.all(rd == (n * (n + 1) / 2 if rank == 1 else rank + 1)), rd
gl = [torch.empty(3) for _ in range(n)] if rank == 0 else None
dist.gather(torch.full((3,), float(rank * 10)), gl, dst=0)
if rank == 0: assert all(torch.all(g == 10.0 * r) for r, g in enumerate(gl))
so = torch.empty(4, dtype=torch.int64)
dist.scatter(so, [torch.full((4,), 100 + r, dtype=torch.int64) for r in range(n)] if rank == 1 else None, src=1)
assert torch.all(so == 100 + rank), so
a2a = torch.empty(n * 2); dist.all_to_all_single(a2a, torch.arange(n * 2).float() + 100 * rank)
assert torch.equal(a2a, torch.cat([torch.arange(2).float() + 2 * rank + 100 * r for r in range(n)])), a2a
lo = [torch.empty(2, 2) for _ in range(n)]
dist.all_to_all(lo, [torch.full((2, 2), float(10 * rank + q)) for q in range(n)])
assert all(torch.all(o == 10.0 * r + rank) for r, o in enumerate(lo)), lo
dist.barrier()
# torch's own DistributedDataParallel on top of the backend
torch.manual_seed(0)
model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 2))
ddp = torch.nn.parallel.DistributedDataParallel(model)
x = torch.randn(4, 8, generator=torch.Generator().manual_seed(rank))
ddp(x).sum().backward()
flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
ref = flat.clone(); dist.all_reduce(ref)
assert torch.allclose(ref / n, flat, atol=1e-6)
print(f"rank {rank} ok", flush=True)
dist.destroy_process_group()
"""

TRAIN_WORKER = r"""
import os, sys, torch
import mccs_b200 as M
from mccs_b200 import models
from mccs_b200.parallel import DataParallel
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"])
torch.manual_seed(0)
m = models.build("gpt2-tiny")
comm = M.Communicator(77, rank, n, device=rank)
ddp = DataParallel(m, comm, bucket_mb=0.05)
opt = torch.optim.SGD(m.parameters(), lr=0.1)
ids = torch.randint(0, 512, (4, 33), generator=torch.Generator().manual_seed(rank))
for it in range(3):
    ddp.zero_grad()
    loss = m(ids[:, :-1], ids[:, 1:])
    loss.backward()
    ddp.finish()
    opt.step()
torch.save([p.detach() for p in m.parameters()], os.environ["OUT"] + f".{rank}")
assert len(ddp.buckets) > 3
ddp.release(); comm.destroy(); M.finalize()
print("ok", flush=True)
"""


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.fixture(params=["events", "memops", "client"])
def standalone_daemon(request):
    """The ways of ordering collectives against the caller: events with completion
    messages, the semaphore protocol (done by the CPU on the host backend), and kernels
    launched by the client library itself (the real kernels on the emulator)."""
    from mccs_b200 import daemon
    d = tempfile.mkdtemp(prefix="mccs-pg-")
    client = request.param == "client"
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=4, listen_port=0,
                       force_host=True, sync="events" if client else request.param,
                       extra='host_kernels = "emulated"\nlaunch = "client"' if client else "")
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    yield sp
    sp.stop()


def _run_workers(code: str, n: int, control: str, extra_env=None):
    env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=control, WORLD_SIZE=str(n), PORT=str(_free_port()),
               MCCS_LOG="warn")
    env.update(extra_env or {})
    procs = [subprocess.Popen([sys.executable, "-c", code], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(n)]
    outs = [p.communicate(timeout=180) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, o + e
    return outs


def test_process_group_two_processes(standalone_daemon):
    _run_workers(WORKER, 2, standalone_daemon.control)

SUBGROUP_WORKER = r"""
import os, torch, torch.distributed as dist
import mccs_b200.process_group as mpg
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"])
dist.init_process_group("mccs", init_method=f"tcp://127.0.0.1:{os.environ['PORT']}", rank=rank, world_size=n)
sub = dist.new_group([0, 2])              # every rank calls new_group, members get a communicator of their own
t = torch.full((5,), float(rank + 1))
if rank in (0, 2):
    dist.all_reduce(t, group=sub)
    assert torch.all(t == 4.0), t
dist.all_reduce(t)
assert torch.all(t == 10.0), t
sub2 = dist.new_group([1, 2])
u = torch.full((3,), float(rank))
if rank in (1, 2):
    dist.broadcast(u, src=2, group=sub2)
    assert torch.all(u == 2.0), u
dist.barrier()
print(f"rank {rank} ok", flush=True)
mpg.shutdown()
dist.destroy_process_group()
"""


def test_process_subgroups(tmp_path):
    """`dist.new_group`: every subgroup is a communicator of its own in the daemon, next to the
    world's; three processes, two overlapping pairs."""
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=4, listen_port=-1, force_host=True)
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        outs = _run_workers(SUBGROUP_WORKER, 3, sp.control)
        assert all(f"rank {r} ok" in o for r, (o, _) in enumerate(outs))
    finally:
        sp.stop()


ACCUM_WORKER = r"""
import os, sys, torch
import mccs_b200 as M
from mccs_b200 import models
from mccs_b200.parallel import DataParallel, ShardedDataParallel
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"])
def batch(r, k):
    return torch.randint(0, 512, (2, 17), generator=torch.Generator().manual_seed(100 * r + k))
torch.manual_seed(0)
m = models.build("gpt2-tiny")
torch.manual_seed(0)
ref = models.build("gpt2-tiny")
comm = M.Communicator(79, rank, n, device=rank)
ddp = DataParallel(m, comm, bucket_mb=0.05)
ddp.zero_grad()
at_start = comm.query()["launched"]       # the parameter broadcast of the constructor
with ddp.no_sync():                       # first micro-batch: accumulate only
    ids = batch(rank, 0); m(ids[:, :-1], ids[:, 1:]).backward(); ddp.finish()
before = comm.query()["launched"]
ids = batch(rank, 1); m(ids[:, :-1], ids[:, 1:]).backward(); ddp.finish()     # second: reduce the sums
assert before == at_start and comm.query()["launched"] - before == len(ddp.buckets), (at_start, before, comm.query()["launched"])
# reference: mean over ranks of the sum over micro-batches
for r in range(n):
    for k in range(2):
        ids = batch(r, k); ref(ids[:, :-1], ids[:, 1:]).backward()
worst = max(float((p.grad - q.grad / n).abs().max()) for p, q in zip(m.parameters(), ref.parameters()))
assert worst < 1e-5, worst
ddp.release(); comm.destroy()
# the sharded form releases cleanly: parameters are ordinary tensors again and still usable
comm = M.Communicator(80, rank, n, device=rank)
z = ShardedDataParallel(m, comm, bucket_mb=0.05)
z.release(); comm.destroy(); M.finalize()
ids = batch(rank, 2); assert torch.isfinite(m(ids[:, :-1], ids[:, 1:]))
print(f"rank {rank} ok", flush=True)
"""


def test_gradient_accumulation_and_release(tmp_path):
    """`DataParallel.no_sync()`: micro-batches inside the block only accumulate, the next
    backward reduces the sums (one AllReduce per bucket for the whole step) and the result is the
    mean over ranks of the summed gradients. `ShardedDataParallel.release()` hands the parameters
    back as ordinary tensors before their buckets are freed."""
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=2, listen_port=-1, force_host=True)
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        outs = _run_workers(ACCUM_WORKER, 2, sp.control)
        assert all(f"rank {r} ok" in o for r, (o, _) in enumerate(outs))
    finally:
        sp.stop()


FSDP_WORKER = r"""
import os, torch, torch.distributed as dist
import mccs_b200.process_group as mpg
from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"])
dist.init_process_group("mccs", init_method=f"tcp://127.0.0.1:{os.environ['PORT']}", rank=rank, world_size=n)
torch.manual_seed(0)
model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
ref = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
ref.load_state_dict(model.state_dict())
f = FSDP(model, device_id=torch.device("cpu"))
opt = torch.optim.SGD(f.parameters(), lr=0.1)
x = torch.randn(8, 16, generator=torch.Generator().manual_seed(rank))
f(x).sum().backward()
opt.step()
# reference: mean gradient over ranks, plain SGD
ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
tot = None
for r in range(n):
    ref.zero_grad()
    ref(torch.randn(8, 16, generator=torch.Generator().manual_seed(r))).sum().backward()
    g = [p.grad.clone() for p in ref.parameters()]
    tot = g if tot is None else [a + b for a, b in zip(tot, g)]
for p, g in zip(ref.parameters(), tot): p.grad = g / n
ropt.step()
with FSDP.summon_full_params(f):
    got = [p.detach().clone() for p in f.parameters()]
want = [p.detach() for p in ref.parameters()]
ok = all(torch.allclose(a.reshape(-1), b.reshape(-1), atol=1e-5) for a, b in zip(got, want))
assert ok
print(f"rank {rank} ok", flush=True)
dist.barrier(); mpg.shutdown(); dist.destroy_process_group()
"""


def test_torch_fsdp_over_the_backend(tmp_path):
    """torch's FullyShardedDataParallel on the backend (all_gather_into_tensor for the
    parameters, reduce_scatter_tensor for the gradients): one SGD step equals the step of a
    plain replica with the mean gradient."""
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=2, listen_port=-1, force_host=True)
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        outs = _run_workers(FSDP_WORKER, 2, sp.control)
        assert all(f"rank {r} ok" in o for r, (o, _) in enumerate(outs))
    finally:
        sp.stop()


ZERO_WORKER = r"""
import os, sys, torch
import mccs_b200 as M
from mccs_b200 import models
from mccs_b200.parallel import ShardedDataParallel
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"])
torch.manual_seed(0)
m = models.build("gpt2-tiny")
total = sum(p.numel() for p in m.parameters())
comm = M.Communicator(78, rank, n, device=rank)
ddp = ShardedDataParallel(m, comm, bucket_mb=0.05)
opt = ddp.make_optimizer(torch.optim.SGD, lr=0.1, momentum=0.9)
ids = torch.randint(0, 512, (4, 33), generator=torch.Generator().manual_seed(rank))
for it in range(3):
    ddp.zero_grad()
    loss = m(ids[:, :-1], ids[:, 1:])
    loss.backward()
    ddp.finish()
    ddp.step(opt)
torch.save([p.detach().clone() for p in m.parameters()], os.environ["OUT"] + f".{rank}")
# the optimizer of this rank holds momentum for about 1/n of the model only
state = sum(v.numel() for st in opt.state.values() for v in st.values() if torch.is_tensor(v))
assert len(ddp.buckets) > 3 and state == ddp.optimizer_state_elements() and state < total * (1.0 / n + 0.2)
assert comm.last_plan()[0] in ("ag_pull", "ag_push", "ag_ring", "ag_nvls")
ddp.release(); comm.destroy(); M.finalize()
print("ok", flush=True)
"""


def test_sharded_data_parallel_matches_single_process(standalone_daemon, tmp_path):
    """ZeRO-1 over the service's ReduceScatter: reduce-scattered gradients, optimizer state for
    1/n of the model per rank, updated parts all-gathered: same parameters as momentum SGD in
    one process on the combined batch, on every rank."""
    import torch
    from mccs_b200 import models
    out = str(tmp_path / "params")
    n = 2
    _run_workers(ZERO_WORKER, n, standalone_daemon.control, {"OUT": out})
    torch.manual_seed(0)
    m = models.build("gpt2-tiny")
    opt = torch.optim.SGD(m.parameters(), lr=0.1, momentum=0.9)
    batches = [torch.randint(0, 512, (4, 33), generator=torch.Generator().manual_seed(r)) for r in range(n)]
    for _ in range(3):
        opt.zero_grad()
        (sum(m(b[:, :-1], b[:, 1:]) for b in batches) / n).backward()
        opt.step()
    for r in range(n):
        got = torch.load(out + f".{r}")
        for a, b in zip(got, m.parameters()):
            assert torch.allclose(a, b.detach(), rtol=1e-4, atol=1e-5)


def test_data_parallel_matches_single_process(standalone_daemon, tmp_path):
    import torch
    from mccs_b200 import models
    out = str(tmp_path / "params")
    n = 2
    _run_workers(TRAIN_WORKER, n, standalone_daemon.control, {"OUT": out})
    torch.manual_seed(0)
    m = models.build("gpt2-tiny")
    opt = torch.optim.SGD(m.parameters(), lr=0.1)
    batches = [torch.randint(0, 512, (4, 33), generator=torch.Generator().manual_seed(r)) for r in range(n)]
    for _ in range(3):
        opt.zero_grad()
        (sum(m(b[:, :-1], b[:, 1:]) for b in batches) / n).backward()
        opt.step()
    for r in range(n):
        got = torch.load(out + f".{r}")
        for a, b in zip(got, m.parameters()):
            assert torch.allclose(a, b.detach(), rtol=1e-4, atol=1e-5)


def test_training_driver_checkpoint_roundtrip(tmp_path):
    """--save then --resume continues from the saved weights: the resumed run's first
    loss equals the loss the first run would have seen next."""
    import json
    import subprocess
    import sys
    from helpers import REPO
    ck = str(tmp_path / "ck.pt")
    env = dict(os.environ, PYTHONPATH=REPO)
    base = [sys.executable, "-m", "mccs_b200.parallel.train", "--model", "gpt2-tiny", "--backend", "none",
            "--batch", "2", "--seq", "32", "--warmup", "1"]
    a = subprocess.run(base + ["--steps", "3", "--save", ck], env=env, capture_output=True, text=True, timeout=300)
    assert a.returncode == 0, a.stderr[-2000:]
    ra = json.loads(a.stdout.strip().splitlines()[-1])
    assert ra["step"] == 4 and os.path.exists(ck)
    b = subprocess.run(base + ["--steps", "1", "--resume", ck], env=env, capture_output=True, text=True, timeout=300)
    assert b.returncode == 0, b.stderr[-2000:]
    rb = json.loads(b.stdout.strip().splitlines()[-1])
    assert rb["step"] == 6
    # same data every step (one synthetic batch), so the loss keeps falling across the restart
    assert rb["first_loss"] < ra["last_loss"] + 1e-3 and rb["first_loss"] < ra["first_loss"]
