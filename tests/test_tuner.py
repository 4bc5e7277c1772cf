"""The tile-shape tuner: selection, cache and persistence on CPU (made-up times); measured
selection on the GPU."""
import json

import numpy as np
import pytest

import helpers as H
from cumm_b200 import tuner as T
from cumm_b200.tensorview.gemm import ConvOpType, ConvParams, ShuffleStrideType


def test_size_bucket_and_keys():
    assert [T.size_bucket(n) for n in (0, 1, 2, 3, 4, 5, 1024, 1025)] == [0, 0, 1, 2, 2, 3, 10, 11]
    f = H.conv_desp(ConvOpType.Forward, 128, 128)
    d = H.conv_desp(ConvOpType.BackwardInput, 128, 128)
    i8 = H.conv_desp(ConvOpType.Forward, 128, 128, int8_inference=True)
    keys = {T.conv_key(x, 150000, 128, 128, 27, "dev") for x in (f, d, i8)}
    assert len(keys) == 3
    assert T.conv_key(f, 150000, 128, 128, 27, "dev") == T.conv_key(f, 140000, 128, 128, 27, "dev")  # same bucket
    assert T.conv_key(f, 150000, 128, 128, 27, "dev") != T.conv_key(f, 150000, 64, 128, 27, "dev")
    assert T.conv_key(f, 150000, 128, 128, 27, "dev") != T.conv_key(f, 150000, 128, 128, 27, "other")


def test_candidates_come_from_the_listed_descriptors():
    assert sorted(T.conv_candidates(H.conv_desp(ConvOpType.Forward, 128, 128))) == [
        (128, 64, 64), (128, 64, 128), (128, 128, 64), (128, 128, 128)]
    assert sorted(T.conv_candidates(H.conv_desp(ConvOpType.BackwardWeight, 128, 128))) == [(128, 64, 128), (128, 128, 128)]
    assert sorted(T.conv_candidates(H.conv_desp(ConvOpType.Forward, 128, 128, int8_inference=True))) == [
        (128, 64, 128), (128, 128, 128)]
    assert len(T.gemm_candidates(H.gemm_desp(ShuffleStrideType.ShuffleAC))) == 4
    assert len(T.gemm_candidates(H.gemm_desp(ShuffleStrideType.ShuffleAB, trans_a=True, trans_b=False))) == 2


def test_selection_cache_and_persistence(tmp_path):
    times = {(128, 64, 64): 30.0, (128, 64, 128): 25.0, (128, 128, 64): 21.0, (128, 128, 128): 22.5}
    calls = []

    def make_launch(tile):
        if tile == (128, 64, 64):
            raise RuntimeError("error: problem not supported by this descriptor (alignment)")
        return lambda: calls.append(tile)

    def timer(launch, stream, warmup, reps):
        launch()
        return times[calls[-1]]

    path = tmp_path / "sub" / "tune.json"
    t = T.Tuner(cache_path=str(path), timer=timer, device_name="fake")
    cands = list(times)
    assert t._select("k1", cands, make_launch, 0) == (128, 128, 64)
    assert t.measurements == 3  # the unsupported variant is skipped, not timed
    blob = json.loads(path.read_text())
    assert blob["entries"]["k1"]["tile_shape"] == [128, 128, 64]
    assert blob["entries"]["k1"]["tried"]["128x128x128"] == 22.5
    # same object: cached
    assert t._select("k1", cands, make_launch, 0) == (128, 128, 64) and t.measurements == 3
    # a new process reads the file and measures nothing
    t2 = T.Tuner(cache_path=str(path), timer=timer, device_name="fake")
    assert t2._select("k1", cands, make_launch, 0) == (128, 128, 64) and t2.measurements == 0
    # a cached shape that is no longer among the candidates is measured again
    assert t2._select("k1", [(128, 64, 128), (128, 128, 128)], make_launch, 0) == (128, 128, 128)
    assert t2.measurements == 2
    # nothing supports the problem
    with pytest.raises(RuntimeError, match="can't find any suitable algo"):
        t2._select("k2", [(128, 64, 64)], make_launch, 0)
    # an unreadable cache file is the same as none
    path.write_text("{not json")
    t3 = T.Tuner(cache_path=str(path), timer=timer, device_name="fake")
    assert t3.entries() == {}


@pytest.mark.gpu
def test_tune_conv_measures_once_and_stays_correct(cuda_lib, oracle, tmp_path):
    import torch
    from cumm_b200 import workloads as W
    from cumm_b200.conv.main import ConvMainUnitTest
    tb, _ = H.random_tables(4000, 901)
    rng = np.random.default_rng(902)
    C = K = 128
    x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
    w = (rng.standard_normal((K, 27, C)) / np.sqrt(27 * C) * 4).astype(np.float16)
    p = ConvParams(3, ConvOpType.Forward)
    p.conv_algo_desp = H.conv_desp(ConvOpType.Forward, C, K)
    p.input, p.weight = H.dev(x, torch), H.dev(w, torch)
    out = torch.zeros((tb.n_out, K), dtype=torch.float16, device="cuda")
    p.output = out
    p.indices, p.mask, p.mask_argsort = H.dev(tb.indices, torch), H.mask_to_torch(tb.mask, torch), H.dev(tb.mask_argsort, torch)
    t = T.Tuner(cache_path=str(tmp_path / "tune.json"), reps=3)
    before = list(p.conv_algo_desp.tile_shape)
    best = t.tune_conv(p)
    assert list(p.conv_algo_desp.tile_shape) == before, "the caller's descriptor is left as it is"
    assert tuple(best.tile_shape) in T.conv_candidates(p.conv_algo_desp)
    assert t.measurements == 4
    entry = next(iter(t.entries().values()))
    assert len(entry["tried"]) == 4 and entry["us"] == min(entry["tried"].values())
    again = T.Tuner(cache_path=str(tmp_path / "tune.json")).tune_conv(p)
    assert again.tile_shape == best.tile_shape
    p.conv_algo_desp = best
    out.zero_()
    ConvMainUnitTest.implicit_gemm2(p)
    torch.cuda.synchronize()
    H.check_status()
    want = oracle.mask_igemm(x, w, np.zeros((tb.n_out, K), np.float16), tb.indices, tb.mask, tb.mask_argsort)
    H.assert_close_f16(out.cpu().numpy(), want, "forward with the tuned descriptor")
