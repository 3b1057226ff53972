"""continuous_count and route on the GPU against the oracle: bit exact."""

import os

import numpy as np
import pytest
import torch

import ck_oracle as orc

pytestmark = pytest.mark.gpu


def _sizes():
    s = set()
    for i in range(0, 15, 2):
        for j in (0, 1, 7):
            s.add(2**i + j)
    s.update([0, 3, 127, 128, 129, 255, 257, 2999, 3517, 100003])
    return sorted(s)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
def test_continuous_count_matches_bincount(dtype):
    """Reference recipe: tests/kernels/continuous_count_test.py:19-41 (randint over 72 values, exact)."""
    from cute_kernels import continuous_count_cute

    for n in _sizes():
        if n == 0:
            continue
        ids = orc.gen_ids(42, n, 72, "uniform", np.int64 if dtype == torch.int64 else np.int32)
        out = continuous_count_cute(torch.from_numpy(ids).cuda(), 72)
        assert out.dtype == torch.uint32
        assert np.array_equal(out.cpu().numpy(), orc.continuous_count_ref(ids, 72)), n


def test_continuous_count_edges():
    from cute_kernels import continuous_count_cute

    x = torch.tensor([0, 5, -1, 9, 3, 3, 100], dtype=torch.int64, device="cuda")
    assert continuous_count_cute(x, 6).cpu().tolist() == [1, 0, 0, 2, 0, 1]  # out of range ignored
    assert continuous_count_cute(x, 1).cpu().tolist() == [7]  # size == 1 shortcut of the reference
    big = orc.gen_ids(1, 50000, 16384, "uniform", np.int32)
    assert np.array_equal(continuous_count_cute(torch.from_numpy(big).cuda(), 16384).cpu().numpy(),
                          orc.continuous_count_ref(big, 16384))
    with pytest.raises(RuntimeError):
        continuous_count_cute(x, 16385)
    # unaligned view (the reference's 128-bit loads would need 16-byte alignment)
    y = torch.from_numpy(orc.gen_ids(3, 1001, 8, "uniform", np.int32)).cuda()
    assert np.array_equal(continuous_count_cute(y[1:], 8).cpu().numpy(), orc.continuous_count_ref(y[1:].cpu().numpy(), 8))


def test_continuous_count_compiled():
    from cute_kernels import continuous_count_cute

    fn = torch.compile(continuous_count_cute, fullgraph=True)
    ids = orc.gen_ids(5, 4097, 72, "uniform", np.int64)
    assert np.array_equal(fn(torch.from_numpy(ids).cuda(), 72).cpu().numpy(), orc.continuous_count_ref(ids, 72))


def _check_route(ids_np, E):
    from cute_kernels import route

    r = route(torch.from_numpy(ids_np).cuda(), E, with_sorted_expert=True)
    ref = orc.route_ref(ids_np, E)
    assert np.array_equal(r.counts.cpu().numpy(), ref["counts"])
    assert np.array_equal(r.excl_offsets.cpu().numpy(), ref["excl_off"])
    assert np.array_equal(r.end_offsets.cpu().numpy(), ref["end_off"])
    assert np.array_equal(r.sorted_idx.cpu().numpy(), ref["sorted_idx"])
    assert np.array_equal(r.sorted_expert.cpu().numpy(), ref["sorted_expert"])
    assert np.array_equal(r.padded_off.cpu().numpy(), ref["padded_off"])
    assert np.array_equal(r.mtile_off.cpu().numpy(), ref["mtile_off"])
    assert np.array_equal(r.row_map.cpu().numpy(), ref["row_map"])


@pytest.mark.parametrize("E", [1, 2, 3, 8, 64, 72, 128, 1024])
def test_route_small_exhaustive(E):
    for n in [0, 1, 2, 31, 32, 33, 127, 128, 129, 255, 256, 300, 1000, 4097]:
        _check_route(orc.gen_ids(n + E, n, E, "uniform", np.int32), E)
        _check_route(orc.gen_ids(n + E, n, E, "zipf", np.int64), E)


def test_route_matches_reference_golden(golden_dir):
    from cute_kernels import route

    g = np.load(os.path.join(golden_dir, "routing.npz"))
    for name in ["u72_i64", "u72_i32", "zipf64", "tiny"]:
        n, E, dist, isz = (int(v) for v in g[f"{name}_meta"])
        ids = orc.gen_ids(7, n, E, "zipf" if dist else "uniform", np.int64 if isz == 8 else np.int32)
        r = route(torch.from_numpy(ids).cuda(), E)
        assert np.array_equal(r.counts.cpu().numpy(), g[f"{name}_counts"])
        assert np.array_equal(r.sorted_idx.cpu().numpy(), g[f"{name}_sorted_idx"])
        assert np.array_equal(r.end_offsets.cpu().numpy(), g[f"{name}_end_off"])


@pytest.mark.parametrize("dist", ["uniform", "zipf"])
@pytest.mark.parametrize("dtype", [np.int32, np.int64])
def test_route_full_size(dist, dtype):
    """16,777,216 ids over 64 experts: bit exact against the oracle."""
    _check_route(orc.gen_ids(0, 1 << 24, 64, dist, dtype), 64)


def test_route_skewed_and_empty_experts():
    ids = np.zeros(5000, dtype=np.int32)  # everything to expert 0, the others empty
    _check_route(ids, 16)
    ids = np.full(777, 15, dtype=np.int64)
    _check_route(ids, 16)


@pytest.mark.expects_dev_status
def test_route_flags_out_of_range_ids():
    import cute_kernels
    from cute_kernels import route

    ids = torch.tensor([0, 1, 9, 1, -3, 2], dtype=torch.int64, device="cuda")
    r = route(ids, 4)
    assert r.counts.cpu().tolist() == [1, 2, 1, 0]
    assert r.sorted_idx.cpu().tolist()[:4] == [0, 1, 3, 5]
    with pytest.raises(RuntimeError, match="CK_DEV_RANGE"):
        cute_kernels.check_device_status()
    cute_kernels.check_device_status()  # cleared
