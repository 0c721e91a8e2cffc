"""The ops enqueue work only (no host synchronisation, no device->host copy, no allocation inside the C ABI), so a
quant -> grouped GEMM sequence can be captured into a CUDA graph and replayed on new data, like the reference's ops."""
import numpy as np
import pytest
import torch

from tests import _cases as C

pytestmark = pytest.mark.gpu


def test_quant_then_gemm_replays_from_a_cuda_graph():
    from expert_specialization_moe_b200 import (es_sm100_mxfp8_blockscaled_grouped_mm as mm,
                                                es_sm100_mxfp8_blockscaled_grouped_quant as quant)
    from oracle import mxfp8_quant_oracle as Q
    dev = "cuda"
    counts, N, K = [3, 0, 200, 40, 130], 256, 512
    inp = C.mxfp8_gemm_inputs(counts, N, K, seed=11)
    T = sum(counts)
    ps, eo, bo, sf_rows = Q.offsets_from_counts(counts, N, K)
    ps, eo, bo = (torch.from_numpy(v).to(dev) for v in (ps, eo, bo))
    x = torch.randn((T, K), device=dev).to(torch.bfloat16)
    a = torch.zeros((T, K), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    sfa = torch.zeros((sf_rows, K // 32), dtype=torch.uint8, device=dev)
    b = torch.from_numpy(inp["w_codes"]).to(dev).view(torch.float8_e4m3fn).transpose(1, 2)
    sfb = torch.from_numpy(inp["sfb"]).to(dev)
    d = torch.zeros((T, N), dtype=torch.bfloat16, device=dev)

    def run():
        quant(x, ps, eo, bo, a, sfa)
        mm(d, a, b, sfa, sfb, ps, eo, bo)

    run()                                   # warm-up outside capture (kernel attributes, tensor-map entry point)
    torch.cuda.synchronize()
    eager = d.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            run()
    d.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(d, eager)
    # new activations in the same buffers: the replay must recompute from them
    x.copy_(torch.randn((T, K), device=dev).to(torch.bfloat16))
    graph.replay()
    torch.cuda.synchronize()
    replayed = d.clone()
    run()
    torch.cuda.synchronize()
    assert torch.equal(replayed, d) and not torch.equal(replayed, eager)
    rc, raw = C.device_status()
    assert rc == 0, raw
