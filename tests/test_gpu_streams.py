"""Launches that overlap on the GPU: a captured forward replayed on one stream while eager
forwards loop on another, and one prepared call launched back to back.  Every prepared call
owns its tile-ticket counters, so two calls never draw tiles from the same counter, whatever
the library's round-robin pool hands to other launches in between; results are checked against
the oracle."""
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


def test_the_same_prepared_call_back_to_back(cuda_lib, oracle):
    """One prepared int8 forward launched many times in a row on one stream, eagerly and from a
    graph: int8 convolutions are launched with programmatic dependent launch, so a launch starts
    drawing tiles while its predecessor -- the same call -- still runs.  The call alternates
    between two pairs of ticket counters; every launch must leave the bit-exact result."""
    import torch
    from cumm_b200.layer import DeviceTables, SparseConvLayer
    grid = (8, 64, 64)
    C = K = 128
    tb = W.build_tables(W.sample_coords(20000, 721, grid), grid=grid, stride=(2, 2, 2), subm=False)
    rng = np.random.default_rng(722)
    x = rng.integers(-127, 128, (tb.n_in, C)).astype(np.int8)
    w = rng.integers(-127, 128, (K, 27, C)).astype(np.int8)
    scale = rng.uniform(1e-3, 1e-2, K).astype(np.float32)
    bias = rng.standard_normal(K).astype(np.float32)
    want = oracle.mask_igemm_s8(x, w, np.zeros((tb.n_out, K), np.int8), scale, bias, tb.indices, tb.mask,
                                tb.mask_argsort)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        out = torch.zeros((tb.n_out, K), dtype=torch.int8, device="cuda")
        L = SparseConvLayer(DeviceTables.from_host(tb, "cuda"), H.dev(w, torch), H.dev(x, torch), out,
                            stream=stream.cuda_stream)
        L.prepare_int8(H.dev(scale, torch), H.dev(bias, torch))
        for _ in range(7):
            L.fwd.launch()
        stream.synchronize()
        H.check_status()
        assert (out.cpu().numpy() == want).all(), "eager launches back to back"
        out.zero_()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for _ in range(5):
                L.fwd.launch()
        for _ in range(3):
            g.replay()
        stream.synchronize()
    H.check_status()
    assert (out.cpu().numpy() == want).all(), "graph of back-to-back launches, replayed"
