"""The allocation-free local AllReduce (csrc/include/mccs_noalloc.h), called through
its exported C symbol, against the service's regular AllReduce on the same inputs.

Who needs the entry point: callers that may not allocate when they reduce — inside a
frozen or exhausted memory pool, in callbacks and latency-critical sections that must
not enter the CUDA allocator. It keeps its synchronisation scratch in a static device
array, so consecutive calls share state; two calls in a row check that the second one
starts from a clean slate. Further cases: free device memory does not move across calls,
the kernels' status words can be read back, and the aliasing rules. This file is collected last on purpose: a failure here
leaves every other test already run."""
import ctypes

import pytest
import torch

from helpers import fresh_comm_id, run_ranks

pytestmark = pytest.mark.gpu

DTYPE_CODE = {torch.float32: 7, torch.float16: 6, torch.bfloat16: 9}


def _entry():
    from mccs_b200 import _lib
    lib = _lib.daemon_lib()
    fn = lib.mccsLocalAllReduceNoAlloc
    fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_size_t,
                   ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def _service_allreduce(M, inputs, dtype):
    """The existing entry point: n ranks on cuda:0 through the daemon, two-shot kernel."""
    n, count, cid = len(inputs), inputs[0].numel(), fresh_comm_id()

    def rank_fn(r):
        torch.cuda.set_device(0)
        with torch.cuda.stream(torch.cuda.Stream()):     # one stream per rank of a communicator
            a, b = M.Buffer(count * 4 + 64, 0), M.Buffer(count * 4 + 64, 0)
            s, d = a.tensor(dtype, count), b.tensor(dtype, count)
            s.copy_(inputs[r])
            c = M.Communicator(cid, r, n, device=0)
            c.all_reduce(s, d, algo="ar_twoshot")
            torch.cuda.synchronize()
            out = d.clone()
            c.destroy()
        return out

    return run_ranks(n, rank_fn)


@pytest.mark.parametrize("dtype,n,count", [(torch.float32, 4, 100003), (torch.bfloat16, 8, 1 << 20), (torch.float16, 2, 4096)])
def test_no_alloc_entry_matches_service(service, dtype, n, count):
    M = service
    assert M.backend() == "cuda"
    fn = _entry()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream()
    tol = 1e-5 if dtype == torch.float32 else 1.6e-2
    for call in range(2):                      # two calls in a row share the static scratch
        g = torch.Generator().manual_seed(50 + call)
        inputs = [((torch.rand(count, generator=g) * 2 - 1).to(dtype)).cuda() for _ in range(n)]
        outputs = [torch.empty_like(x) for x in inputs]
        ins = (ctypes.c_void_p * n)(*[x.data_ptr() for x in inputs])
        outs = (ctypes.c_void_p * n)(*[x.data_ptr() for x in outputs])
        rc = fn(ins, outs, n, count, DTYPE_CODE[dtype], ctypes.c_void_p(stream.cuda_stream))
        assert rc == 0, f"cudaError {rc}"
        torch.cuda.synchronize()
        want = _service_allreduce(M, inputs, dtype)
        ref = torch.stack([x.double() for x in inputs]).sum(0)
        for r in range(n):
            assert torch.allclose(outputs[r].double(), want[r].double(), rtol=tol, atol=tol * n)
            assert torch.allclose(outputs[r].double(), ref, rtol=tol, atol=tol * n)


class _Status(ctypes.Structure):
    _fields_ = [("error", ctypes.c_uint * 8), ("peer", ctypes.c_uint * 8)]


def test_no_alloc_entry_allocates_nothing_and_reports_status(service):
    """The property the entry point exists for: once the set-up call has run, calls take no
    device memory (free memory as the driver reports it and PyTorch's own counters are the
    same before and after), and what the kernels reported can be read back."""
    from mccs_b200 import _lib
    lib = _lib.daemon_lib()
    fn = _entry()
    torch.cuda.set_device(0)
    assert lib.mccsLocalAllReduceNoAllocPrepare() == 0
    n, count = 4, 1 << 20
    xs = [torch.full((count,), float(r + 1), device="cuda") for r in range(n)]
    ys = [torch.empty_like(x) for x in xs]
    ins = (ctypes.c_void_p * n)(*[x.data_ptr() for x in xs])
    outs = (ctypes.c_void_p * n)(*[y.data_ptr() for y in ys])
    stream = torch.cuda.current_stream()
    st = _Status()
    lib.mccsLocalAllReduceNoAllocStatus.argtypes = [ctypes.POINTER(_Status), ctypes.c_void_p]
    assert fn(ins, outs, n, count, 7, ctypes.c_void_p(stream.cuda_stream)) == 0      # every kernel has run once
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(5):
        assert fn(ins, outs, n, count, 7, ctypes.c_void_p(stream.cuda_stream)) == 0
    assert lib.mccsLocalAllReduceNoAllocStatus(ctypes.byref(st), ctypes.c_void_p(stream.cuda_stream)) == 0
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"device memory in use changed by {free0 - free1} bytes"
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == (alloc0, reserved0)
    assert list(st.error) == [0] * 8 and list(st.peer) == [0] * 8
    assert all(bool(torch.all(y == 10.0)) for y in ys)


def test_no_alloc_entry_aliasing_rules(service):
    """Any output may be exactly one of the inputs; partial overlaps are refused."""
    fn = _entry()
    torch.cuda.set_device(0)
    count = 4096
    a = torch.arange(count, dtype=torch.float32, device="cuda")
    b = torch.ones(count + 64, dtype=torch.float32, device="cuda")
    want = (a + 1).clone()
    # crossed: out[0] is in[1] and out[1] is in[0]
    ins = (ctypes.c_void_p * 2)(a.data_ptr(), b.data_ptr())
    outs = (ctypes.c_void_p * 2)(b.data_ptr(), a.data_ptr())
    assert fn(ins, outs, 2, count, 7, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(a, want) and torch.equal(b[:count], want)
    # an output that starts inside an input, and two outputs sharing their range
    shifted = (ctypes.c_void_p * 2)(b.data_ptr() + 64, a.data_ptr())
    assert fn(ins, shifted, 2, count, 7, None) != 0
    same_out = (ctypes.c_void_p * 2)(a.data_ptr(), a.data_ptr())
    assert fn(ins, same_out, 2, count, 7, None) != 0
    torch.cuda.synchronize()


def test_no_alloc_entry_rejects_what_it_cannot_do(service):
    fn = _entry()
    torch.cuda.set_device(0)
    x = torch.zeros(16, device="cuda")
    one = (ctypes.c_void_p * 1)(x.data_ptr())
    many = (ctypes.c_void_p * 9)(*([x.data_ptr()] * 9))
    assert fn(many, many, 9, 16, 7, None) != 0        # more buffers than the scratch has slots for
    assert fn(one, one, 1, 16, 2, None) != 0          # int32 is not offered
    assert fn(one, one, 0, 16, 7, None) != 0
    assert fn(one, one, 1, 16, 7, None) == 0          # single buffer in place: nothing to do, still valid
    torch.cuda.synchronize()


def test_ops_binding_of_the_no_alloc_entry(service):
    """The same entry point through `mccs_b200.ops`, in place, and its argument checks."""
    from mccs_b200 import ops
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(5)
    xs = [(torch.rand(70001, generator=g) * 2 - 1).cuda() for _ in range(3)]
    ref = torch.stack([x.double() for x in xs]).sum(0)
    outs = ops.local_all_reduce_no_alloc(xs)
    torch.cuda.synchronize()
    assert all(o is x for o, x in zip(outs, xs))
    for x in xs:
        assert torch.allclose(x.double(), ref, rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError):
        ops.local_all_reduce_no_alloc([torch.zeros(4, device="cuda", dtype=torch.int32)])
    with pytest.raises(ValueError):
        ops.local_all_reduce_no_alloc([torch.zeros(4, device="cuda"), torch.zeros(5, device="cuda")])
