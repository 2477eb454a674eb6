"""The network object of the C ABI (``lc0b200_net_*``): the whole forward pass driven from C.

It must give what ``net.Bt4Net`` gives (the same kernels in the same order; only the upload-time
LayerNorm folding is summed in another order) and meet the fp32 oracle's tolerance on its own.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from oracle import bt4_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg():
    from lczero_triton_b200 import build

    build.build()
    from lczero_triton_b200 import _lib, config, mapping_table, native, net, synthetic, weights

    return {"config": config, "net": net, "native": native, "synthetic": synthetic, "weights": weights, "lib": _lib,
            "table": torch.tensor(mapping_table.values(), dtype=torch.int32)}


def _within_tolerance(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    err = (got - want).abs()
    return (err <= 1e-2) | (err <= 1e-2 * want.abs())


def _no_timeouts(pkg) -> None:
    status, detail = pkg["lib"].device_status()
    assert status == 0, f"a kernel gave up: {detail}"


@pytest.mark.parametrize("batch", [1, 5, 32])
def test_tiny_network_through_the_c_object(pkg, batch) -> None:
    cfg = pkg["config"].TINY
    weights = pkg["weights"].random_weights(cfg, 3)
    masks, values = pkg["synthetic"].synthetic_planes(batch, 3)
    native = pkg["native"].NativeNet(weights, cfg, max_batch=32)
    policy, wdl, mlh = (x.cpu() for x in native.forward(masks.cuda(), values.cuda()))
    _no_timeouts(pkg)
    want_policy, want_wdl, want_mlh = O.forward(weights, cfg, masks, values, table=pkg["table"])
    assert _within_tolerance(policy, want_policy).all()
    assert _within_tolerance(wdl, want_wdl).all()
    assert _within_tolerance(mlh, want_mlh).all()
    # against the Python-driven network: same kernels, same order
    ref = pkg["net"].Bt4Net(weights, cfg)
    ref_policy, ref_wdl, ref_mlh = (x.cpu() for x in ref.forward(masks.cuda(), values.cuda()))
    torch.testing.assert_close(policy, ref_policy, rtol=2e-2, atol=2e-3)
    torch.testing.assert_close(wdl, ref_wdl, rtol=2e-2, atol=2e-3)
    torch.testing.assert_close(mlh, ref_mlh, rtol=2e-2, atol=2e-3)
    native.close()


def test_bt4_shape_through_the_c_object_matches_the_python_network(pkg) -> None:
    cfg = pkg["config"].BT4
    batch = 8
    weights = pkg["weights"].random_weights(cfg, 0)
    masks, values = pkg["synthetic"].synthetic_planes(batch, 0)
    native = pkg["native"].NativeNet(weights, cfg, max_batch=16)
    got = [x.cpu() for x in native.forward(masks.cuda(), values.cuda())]
    # a second call reuses the workspace and must reproduce the first bit for bit
    again = [x.cpu() for x in native.forward(masks.cuda(), values.cuda())]
    _no_timeouts(pkg)
    for a, b in zip(got, again):
        assert torch.equal(a, b)
    # Two bf16 evaluations of fifteen layers differ by rounding flips that the layers amplify (the folded
    # LayerNorm vectors are summed in another order): hold both to the oracle's bound, and each other to
    # half of it.
    ref = pkg["net"].Bt4Net(weights, cfg)
    python_net = [x.cpu() for x in ref.forward(masks.cuda(), values.cuda())]
    want = O.forward(weights, cfg, masks, values, table=pkg["table"])
    for a, b, w in zip(got, python_net, want):
        spread = float(w.std().clamp_min(1e-6))
        assert _within_tolerance(a, w).all()
        assert float((a - w).abs().max()) < 0.3 * spread
        assert float((a - b).abs().max()) < 0.15 * spread + 2e-3
    native.close()


@pytest.mark.parametrize("batch", [15, 30, 77])
def test_bt4_row_counts_that_leave_a_cta_pair_half_empty(pkg, batch) -> None:
    """960, 1920 and 4928 token rows: the 256-wide GEMM tiles run as 256-row tiles of two CTAs, and the last tile
    of each GEMM is ragged (only part of the first CTA's rows, or of the second's, exist).  Every position
    against the fp32 oracle, against the last positions run alone, and bit for bit against the same positions as the
    tail of a larger batch."""
    cfg = pkg["config"].BT4
    weights = pkg["weights"].random_weights(cfg, 4)
    masks, values = pkg["synthetic"].synthetic_planes(batch, 4)
    native = pkg["native"].NativeNet(weights, cfg, max_batch=batch)
    got = [x.cpu() for x in native.forward(masks.cuda(), values.cuda())]
    _no_timeouts(pkg)
    native.close()
    want = O.forward(weights, cfg, masks, values, table=pkg["table"])
    rounded = O.forward(weights, cfg, masks, values, table=pkg["table"], round_to=torch.bfloat16)
    for a, w, r in zip(got, want, rounded):
        err, floor = float((a - w).abs().max()), float((r - w).abs().max())
        assert err <= 1.5e-2 and err <= 2.0 * floor + 2e-3, (err, floor)
    # Positions are independent: the last three alone give the same numbers up to bf16 rounding flips (a batch of
    # three runs narrow GEMM tiles, whose epilogue combines its per-column vectors in another order than the wide
    # tiles'; from 15 positions up every batch size gives the same bits, which the next lines hold for 16 more).
    alone = pkg["native"].NativeNet(weights, cfg, max_batch=3)
    tail = [x.cpu() for x in alone.forward(masks[-3:].cuda(), values[-3:].cuda())]
    alone.close()
    for a, b, w in zip(got, tail, want):
        assert float((a[-3:] - b).abs().max()) < 0.15 * float(w.std().clamp_min(1e-6)) + 2e-3
    wider = pkg["native"].NativeNet(weights, cfg, max_batch=batch + 16)
    more_masks, more_values = pkg["synthetic"].synthetic_planes(batch + 16, 9)
    more_masks[-batch:], more_values[-batch:] = masks, values
    again = [x.cpu() for x in wider.forward(more_masks.cuda(), more_values.cuda())]
    wider.close()
    for a, b in zip(got, again):
        assert torch.equal(a, b[-batch:])


@pytest.mark.parametrize("name", ["TINY", "BT4"])
def test_int8_mode_through_the_c_object_equals_the_python_network(pkg, name) -> None:
    """int8 GEMMs, stand-alone LayerNorms: nothing is summed differently on the two sides (the weights
    are quantised by the same rule, on the device here and on the host there), so the outputs agree
    bit for bit."""
    cfg = getattr(pkg["config"], name)
    batch = 6
    weights = pkg["weights"].random_weights(cfg, 2)
    masks, values = pkg["synthetic"].synthetic_planes(batch, 2)
    native = pkg["native"].NativeNet(weights, cfg, max_batch=8, mode="int8")
    got = [x.cpu() for x in native.forward(masks.cuda(), values.cuda())]
    _no_timeouts(pkg)
    ref = pkg["net"].Bt4Net(weights, cfg, mode="int8", deferred_layer_norm=False)  # the object's int8 tower
    want = [x.cpu() for x in ref.forward(masks.cuda(), values.cuda())]
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    native.close()


def test_object_rejects_misuse(pkg) -> None:
    lib = pkg["lib"].load()
    cfg = pkg["config"].TINY
    cfg_c = pkg["native"].NetConfigC.from_config(cfg)
    nbytes = lib.lc0b200_net_arena_bytes(ctypes.byref(cfg_c), 4)
    assert nbytes > 0
    arena = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    handle = ctypes.c_void_p()
    assert lib.lc0b200_net_create(ctypes.byref(handle), ctypes.byref(cfg_c), 4, arena.data_ptr(), nbytes - 4096) == 7
    assert lib.lc0b200_net_create(ctypes.byref(handle), ctypes.byref(cfg_c), 4, arena.data_ptr(), nbytes) == 0
    host = torch.zeros(16, dtype=torch.bfloat16)
    assert lib.lc0b200_net_set_weight(handle, b"/no/such/buffer", host.data_ptr(), 16, None) == 3
    assert lib.lc0b200_net_set_weight(handle, b"/attn_body/add/w", host.data_ptr(), 16, None) == 2
    assert lib.lc0b200_net_finalize(handle, None) == 1          # weights missing
    out = torch.empty(4 * 1858, dtype=torch.float32, device="cuda")
    planes = torch.zeros((4, 112), dtype=torch.int64, device="cuda")
    assert lib.lc0b200_net_forward(handle, planes.data_ptr(), planes.data_ptr(), 4, out.data_ptr(), out.data_ptr(),
                                   out.data_ptr(), None) == 3  # not finalised
    lib.lc0b200_net_destroy(handle)
    bad = pkg["native"].NetConfigC.from_config(cfg)
    bad.heads = 3
    assert lib.lc0b200_net_arena_bytes(ctypes.byref(bad), 4) == 0


@pytest.mark.parametrize("mode", ["bf16", "int8"])
@pytest.mark.parametrize(("cfg_name", "batch"), [("TINY", 32), ("BT4", 64), ("BT4", 192)])
def test_replayed_graph_and_back_to_back_launches_equal_one_forward(pkg, cfg_name, batch, mode) -> None:
    """The forward as the benchmark runs it: captured once into a CUDA graph and replayed.  Every kernel may be
    scheduled while its predecessor on the stream is still running (programmatic dependent launch) and waits
    for it before touching memory; a kernel that touched memory too early would show here as results that depend
    on timing: five launches in a row, a graph replay, and a replay on new planes written into the same input
    buffers must each equal one forward on its own, bit for bit."""
    cfg = getattr(pkg["config"], cfg_name)
    weights = pkg["weights"].random_weights(cfg, 5)
    net = pkg["native"].NativeNet(weights, cfg, max_batch=batch, mode=mode)
    masks, values = (x.cuda() for x in pkg["synthetic"].synthetic_planes(batch, 5))
    other_masks, other_values = (x.cuda() for x in pkg["synthetic"].synthetic_planes(batch, 6))
    alone = [x.clone() for x in net.forward(masks, values)]
    torch.cuda.synchronize()
    other_alone = [x.clone() for x in net.forward(other_masks, other_values)]
    torch.cuda.synchronize()
    assert not torch.equal(alone[0], other_alone[0])
    for _ in range(5):
        again = net.forward(masks, values)
    assert all(torch.equal(a, b) for a, b in zip(alone, again))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = net.forward(masks, values)
    for _ in range(3):
        graph.replay()
    assert all(torch.equal(a, b) for a, b in zip(alone, captured))
    masks.copy_(other_masks)
    values.copy_(other_values)
    graph.replay()
    assert all(torch.equal(a, b) for a, b in zip(other_alone, captured))
    _no_timeouts(pkg)
    net.close()
