"""ck_route_static: routing for hosts that cannot hand the library a workspace.

Some callers of this library sit where no device allocation is possible -- a server whose memory pool is
sealed once it starts serving, a plug-in inside an engine that owns the whole device and passes only the
input and output buffers, a latency-bound step that must not hit the device-wide synchronisation of
cudaMalloc.  For them the library carries a fixed scratch array of its own.  This test drives that entry
point straight through the C ABI, twice in a row on different inputs (the array is shared and keeps the
previous call's contents), and requires the very same bytes as ck_route with a caller workspace.
Collected last on purpose: a failure here cannot hide a failure anywhere else under `pytest -x`.
"""

import numpy as np
import pytest
import torch

import ck_oracle as orc

pytestmark = pytest.mark.gpu


def _buffers(n, E, dev):
    from cute_kernels import _lib

    i32 = dict(dtype=torch.int32, device=dev)
    cap = _lib.lib.ck_route_padded_capacity(n, E)
    return dict(counts=torch.full((E,), 7, dtype=torch.uint32, device=dev), excl=torch.full((E,), -5, **i32),
                end=torch.full((E,), -5, **i32), sidx=torch.full((n,), -5, **i32), sexp=torch.full((n,), -5, **i32),
                poff=torch.full((E + 1,), -5, **i32), moff=torch.full((E + 1,), -5, **i32),
                rmap=torch.full((cap,), -5, **i32))


def _call(static, ids, E):
    from cute_kernels import _lib

    dev = ids.device
    b = _buffers(ids.numel(), E, dev)
    status = _lib.status_word(dev)
    stream = torch.cuda.current_stream().cuda_stream
    common = (ids.data_ptr(), int(ids.dtype == torch.int64), ids.numel(), E, b["counts"].data_ptr(), b["excl"].data_ptr(),
              b["end"].data_ptr(), b["sidx"].data_ptr(), b["sexp"].data_ptr(), b["poff"].data_ptr(), b["moff"].data_ptr(),
              b["rmap"].data_ptr())
    if static:
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        st = _lib.lib.ck_route_static(*common, status.data_ptr(), stream)
        torch.cuda.synchronize()
        # every buffer above was allocated before this bracket: the entry point itself must not change the device's
        # free memory (the first call on a device only looks up the address of the in-library array)
        assert torch.cuda.mem_get_info()[0] == free_before, "ck_route_static changed the device's free memory"
    else:
        ws = torch.empty(_lib.lib.ck_route_workspace_bytes(ids.numel(), E), dtype=torch.uint8, device=dev)
        st = _lib.lib.ck_route(*common, ws.data_ptr(), ws.numel(), status.data_ptr(), stream)
    torch.cuda.synchronize()
    return st, b


def test_route_static_equals_route_on_two_calls_in_a_row():
    cases = [(orc.gen_ids(1, 262144, 64, "zipf", np.int64), 64),   # the fine-grained layer's routed rows
             (orc.gen_ids(2, 32768, 8, "uniform", np.int32), 8),   # smaller and different: stale scratch must not leak
             (orc.gen_ids(3, 100, 128, "uniform", np.int32), 128)]
    for ids_np, E in cases:
        ids = torch.from_numpy(ids_np).cuda()
        st_s, got = _call(True, ids, E)
        st_r, exp = _call(False, ids, E)
        assert st_s == 0 and st_r == 0
        for key in exp:
            assert torch.equal(got[key], exp[key]), key
        ref = orc.route_ref(ids_np, E)
        assert np.array_equal(got["sidx"].cpu().numpy(), ref["sorted_idx"])
        assert np.array_equal(got["counts"].cpu().numpy(), ref["counts"])
        assert np.array_equal(got["rmap"].cpu().numpy(), ref["row_map"])


def test_route_static_rejects_sizes_beyond_its_scratch():
    from cute_kernels import _lib

    limit = _lib.lib.ck_route_static_max_bytes()
    assert limit == 256 + 148 * 32 * 32 * 4
    n, E = 1 << 22, 1024
    assert _lib.lib.ck_route_workspace_bytes(n, E) > limit
    ids = torch.zeros(n, dtype=torch.int32, device="cuda")
    st, b = _call(True, ids, E)
    assert st == -2  # CK_ERR_RANGE, and nothing was launched:
    assert (b["counts"] == 7).all() and (b["sidx"] == -5).all()
    assert _lib.lib.ck_status_string(st) == b"CK_ERR_RANGE"
