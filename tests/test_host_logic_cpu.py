"""Host-side bookkeeping that needs no GPU: the producers' hand-over registry and saved-tensor keys."""
import pytest
import torch

from flame_b200 import checkpoint as ckpt
from flame_b200 import fused_producers as fp


def test_producer_registry_hands_codes_out_once_and_only_for_the_same_tensor():
    t = torch.zeros(256, dtype=torch.bfloat16)
    codes, scales = torch.zeros(256, dtype=torch.uint8), torch.zeros(2)
    assert fp.emitting() == 0 and fp.take(t) is None
    with fp.emit_codes(2):
        assert fp.emitting() == 2
        fp._READY[(t.data_ptr(), t.numel())] = (t._version, codes, scales, t)
        other = torch.zeros(256, dtype=torch.bfloat16)
        assert fp.take(other) is None                       # another tensor: another address
        got = fp.take(t)
        assert got is not None and got[0] is codes and got[1] is scales
        assert fp.take(t) is None                           # once
        fp._READY[(t.data_ptr(), t.numel())] = (t._version, codes, scales, t)
        t.add_(1)                                           # modified since the codes were written: they are stale
        assert fp.take(t) is None
        fp._READY[(t.data_ptr(), t.numel())] = (t._version, codes, scales, t)
        with fp.emit_codes(0):                              # a nested block that must not emit
            assert fp.emitting() == 0
        assert fp.emitting() == 2 and len(fp._READY) == 1   # the inner block does not clear the outer one's records
    assert fp.emitting() == 0 and not fp._READY             # what nobody took is dropped with the block


def test_dense_permutation_and_offloadable_rules():
    x = torch.zeros(2, 3, 4, 5)
    assert ckpt.dense_permutation(x) == (0, 1, 2, 3)
    assert ckpt.dense_permutation(x.transpose(1, 2)) == (0, 2, 1, 3)
    assert x.transpose(1, 2).permute(ckpt.dense_permutation(x.transpose(1, 2))).is_contiguous()
    assert ckpt.dense_permutation(x[:, :, ::2]) is None     # a strided slice is not dense memory
    assert ckpt.dense_permutation(x[:, 1]) == (0, 1, 2) or ckpt.dense_permutation(x[:, 1]) is None
    # CPU tensors, parameters and their views, small and non-BF16 tensors stay where they are
    p = torch.nn.Parameter(torch.zeros(1024, 1024, dtype=torch.bfloat16))
    assert not ckpt.offloadable(p, 1) and not ckpt.offloadable(p.t(), 1)
    assert not ckpt.offloadable(torch.zeros(1 << 20, dtype=torch.bfloat16, requires_grad=True), 1)      # not on a GPU


def test_without_a_pool_the_offload_arm_is_the_recompute_arm_on_cpu():
    lin = torch.nn.Linear(8, 8)
    x = torch.randn(4, 8, requires_grad=True)
    ckpt.clear_activation_offload_pool()
    y = ckpt.checkpoint_offload([x], lambda t: lin(t).relu())
    y.sum().backward()
    g1 = x.grad.clone()
    x.grad = None
    lin(x).relu().sum().backward()
    assert torch.equal(g1, x.grad)
    assert ckpt.activation_offload_pool() is None


def test_bench_host_helpers_need_no_gpu():
    """bench.py's helpers that read the host: available memory, the PCIe description of a device that is not there,
    and the table of pool settings swept under shared links."""
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    avail = bench.host_mem_available_bytes()
    assert avail is None or avail > (1 << 20)
    info = bench.pcie_info(torch, 0)
    assert isinstance(info, dict) and ("error" in info or "bdf" in info)
    labels = [row[0] for row in bench.LINKSWEEP]
    assert len(set(labels)) == len(labels) and labels[0].startswith("default")
    for _, chunk_mb, flags, piece_mb, tile_chunks in bench.LINKSWEEP:
        assert (chunk_mb << 20) % (64 << 10) == 0 and flags in (0, 1, 4) and piece_mb >= 0 and tile_chunks >= 1
    comp, deq = bench.roofline_entries("int8", q_ms=1.0, d_ms=2.0, elems=1 << 20, launches=4)
    assert comp["bound"] == deq["bound"] == "hbm" and comp["achieved"] == round(3.03125 * (1 << 20) / 1e-3 * 1e-9, 1)
    assert comp["frac"] == round(comp["achieved"] / comp["peak"], 4) and deq["achieved"] * 2 == pytest.approx(comp["achieved"], rel=1e-3)
