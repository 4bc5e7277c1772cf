"""Launches that overlap on the GPU: a captured forward replayed on one stream while eager
forwards loop on another.  Every prepared call owns its tile-ticket counters, so the two
never draw tiles from the same counter, whatever the library's round-robin pool hands to
other launches in between; both results are checked against the oracle."""
import numpy as np
import pytest

import helpers as H
from cumm_b200 import workloads as W

pytestmark = pytest.mark.gpu


def test_graph_replay_beside_eager_launches(cuda_lib, oracle):
    import torch
    from cumm_b200.layer import DeviceTables, SparseConvLayer
    grid = (8, 48, 48)
    C = K = 64
    layers, wants, outs = [], [], []
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for i, n in enumerate((9000, 7000)):
        tb = W.build_tables(W.sample_coords(n, 700 + i, grid), grid=grid)
        rng = np.random.default_rng(710 + i)
        x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
        w = (rng.standard_normal((K, 27, C)) / 16).astype(np.float16)
        out = torch.zeros((tb.n_out, K), dtype=torch.float16, device="cuda")
        with torch.cuda.stream(streams[i]):
            layers.append(SparseConvLayer(DeviceTables.from_host(tb, "cuda"), H.dev(w, torch), H.dev(x, torch), out,
                                          stream=streams[i].cuda_stream))
        outs.append(out)
        wants.append(oracle.mask_igemm(x, w, np.zeros((tb.n_out, K), np.float16), tb.indices, tb.mask, tb.mask_argsort))
    torch.cuda.synchronize()
    a, b = layers
    with torch.cuda.stream(streams[0]):
        a.fwd.launch()
        streams[0].synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=streams[0]):
            for _ in range(4):
                a.fwd.launch()
    for rounds in range(20):
        with torch.cuda.stream(streams[0]):
            g.replay()
        with torch.cuda.stream(streams[1]):
            for _ in range(6):
                b.fwd.launch()
        if rounds % 5 == 4:
            # launches of other calls in between advance the library's own pool of counters
            with torch.cuda.stream(streams[1]):
                H.run_conv_fwd(torch, np.zeros((8, C), np.float16), np.zeros((K, 27, C), np.float16),
                               W.build_tables(W.sample_coords(8, 1, grid), grid=grid))
    torch.cuda.synchronize()
    H.check_status()
    H.assert_close_f16(outs[0].cpu().numpy(), wants[0], "captured forward replayed beside eager launches")
    H.assert_close_f16(outs[1].cpu().numpy(), wants[1], "eager forward beside graph replays")
