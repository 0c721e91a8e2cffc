"""es_b200_ep_route_count_static: the routing histogram for callers that cannot hand the library scratch memory
(a server whose allocator owns the whole GPU; an FFI binding that only receives raw pointers).  Its counters live in a
static device array inside the library.  The test calls it through the C ABI twice in a row — the second time with
different ids, fewer experts and fewer pairs, so that whatever the first call left in the shared array is in the way —
and requires exactly the results of es_b200_ep_route_count with caller-provided scratch (integers: equality).
Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, ids, num_experts):
    dev = ids.device
    pairs = ids.numel()
    stream = torch.cuda.current_stream(dev).cuda_stream
    out = {}
    for name in ("scratch", "static"):
        base = torch.full((256, num_experts), -1, dtype=torch.int32, device=dev)
        counts = torch.full((1, num_experts), -1, dtype=torch.int32, device=dev)      # world of one: my own matrix
        table = (ctypes.c_void_p * 1)(counts.data_ptr())
        if name == "scratch":
            scratch = torch.empty((256, num_experts), dtype=torch.int32, device=dev)
            rc = lib.es_b200_ep_route_count(ids.data_ptr(), 1, pairs, num_experts, scratch.data_ptr(),
                                            base.data_ptr(), table, 0, 1, stream)
        else:
            rc = lib.es_b200_ep_route_count_static(ids.data_ptr(), 1, pairs, num_experts, base.data_ptr(), table, 0,
                                                   1, stream)
        assert rc == 0, lib.es_b200_last_error().decode()
        torch.cuda.synchronize(dev)
        out[name] = (base.cpu(), counts.cpu())
    return out


def test_static_scratch_route_count_matches_the_scratch_version_twice():
    from expert_specialization_moe_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(5)
    for num_experts, tokens, topk in [(256, 4096, 8), (96, 517, 3)]:
        ids = torch.randint(0, num_experts, (tokens, topk), generator=g, device=dev, dtype=torch.int64)
        res = _both(lib, ids, num_experts)
        assert torch.equal(res["static"][0], res["scratch"][0]), "segment prefixes differ"
        assert torch.equal(res["static"][1], res["scratch"][1]), "per-expert totals differ"
        want = torch.bincount(ids.reshape(-1).cpu(), minlength=num_experts).to(torch.int32)
        assert torch.equal(res["static"][1][0], want)


def test_static_scratch_route_count_allocates_no_device_memory():
    """The point of the entry point: a call takes no device memory from anybody.  The driver's free-memory figure is
    the same before and after a call (the first call on the device, which looks up the static array's address, was
    made by the test above or is made here before the measurement)."""
    from expert_specialization_moe_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    ids = torch.randint(0, 64, (512, 4), device=dev, dtype=torch.int64)
    base = torch.empty((256, 64), dtype=torch.int32, device=dev)
    counts = torch.empty((1, 64), dtype=torch.int32, device=dev)
    table = (ctypes.c_void_p * 1)(counts.data_ptr())
    stream = torch.cuda.current_stream(dev).cuda_stream
    call = lambda: lib.es_b200_ep_route_count_static(ids.data_ptr(), 1, ids.numel(), 64, base.data_ptr(), table, 0, 1, stream)
    assert call() == 0
    torch.cuda.synchronize(dev)
    free_before, _ = torch.cuda.mem_get_info(dev)
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize(dev)
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before
    assert torch.equal(counts[0].cpu(), torch.bincount(ids.reshape(-1).cpu(), minlength=64).to(torch.int32))


def test_static_scratch_route_count_rejects_more_experts_than_it_holds():
    from expert_specialization_moe_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    ids = torch.zeros((4, 2), dtype=torch.int64, device=dev)
    base = torch.empty((256, 512), dtype=torch.int32, device=dev)
    counts = torch.empty((1, 512), dtype=torch.int32, device=dev)
    table = (ctypes.c_void_p * 1)(counts.data_ptr())
    rc = lib.es_b200_ep_route_count_static(ids.data_ptr(), 1, 8, 512, base.data_ptr(), table, 0, 1,
                                           torch.cuda.current_stream(dev).cuda_stream)
    assert rc != 0 and b"at most 256 experts" in lib.es_b200_last_error()
