"""Row IO by raw address and the row-wise sparse optimizers: CPU contract, GPU kernels against it, stray addresses."""
import pytest
import torch

from recsdk_b200.ops import _lib
from recsdk_b200.ops.by_address import embedding_lookup_by_address, embedding_update_by_address, lazy_adam, sgd


def _scenario(device):
    g = torch.Generator().manual_seed(2)
    table = torch.randn(40, 12, generator=g).to(device)
    before = table.clone()
    rows = torch.tensor([3, 17, 3, 39])
    base = table.data_ptr()
    addr = (base + rows * 12 * 4).to(device)
    addr[1] = 0                                                        # address 0: skipped / zeros
    got = embedding_lookup_by_address(addr, 12, table)
    assert torch.equal(got[0].cpu(), before[3].cpu()) and torch.equal(got[3].cpu(), before[39].cpu()) and float(got[1].abs().sum()) == 0
    vals = torch.randn(4, 12, generator=g).to(device)
    embedding_update_by_address(addr, vals, 0, table)                  # add; row 3 is listed twice
    want = before.clone()
    want[3] += vals[0] + vals[2]
    want[39] += vals[3]
    assert torch.allclose(table.cpu(), want.cpu(), atol=1e-6)
    embedding_update_by_address(addr[3:], vals[:1], 1, table)          # assign
    want[39] = vals[0]
    assert torch.allclose(table.cpu(), want.cpu(), atol=1e-6)
    # optimizers
    var = torch.randn(30, 8, generator=g).to(device)
    m, v = torch.zeros_like(var), torch.zeros_like(var)
    ref_var, ref_m, ref_v = var.clone().cpu(), m.clone().cpu(), v.clone().cpu()
    idx = torch.tensor([5, 9, 5, 0]).to(device)
    gr = torch.randn(4, 8, generator=g).to(device)
    sgd(gr, idx, var, 0.1)
    ref_var.index_add_(0, idx.cpu(), gr.cpu(), alpha=-0.1)
    assert torch.allclose(var.cpu(), ref_var, atol=1e-6)
    sgd(gr, idx, var, 0.1, weight_decay=0.5)
    u = torch.tensor([0, 5, 9])
    gs = torch.stack([gr.cpu()[3], gr.cpu()[0] + gr.cpu()[2], gr.cpu()[1]])
    ref_var[u] -= 0.1 * (gs + 0.5 * ref_var[u])
    assert torch.allclose(var.cpu(), ref_var, atol=1e-6)
    lazy_adam(gr, idx, m, v, var, 0.01, 0.9, 0.999, 1e-8)
    ref_m[u] = 0.1 * gs
    ref_v[u] = 0.001 * gs * gs
    ref_var[u] -= 0.01 * ref_m[u] / (ref_v[u].sqrt() + 1e-8)
    assert torch.allclose(var.cpu(), ref_var, atol=1e-5) and torch.allclose(m.cpu(), ref_m, atol=1e-7)
    assert float(m.cpu()[1].abs().sum()) == 0                          # untouched rows keep their moments
    return table


def test_by_address_and_sparse_optimizers_cpu():
    table = _scenario("cpu")
    with pytest.raises(IndexError):
        embedding_lookup_by_address(torch.tensor([table.data_ptr() + table.numel() * 4]), 12, table)


@pytest.mark.gpu
def test_by_address_and_sparse_optimizers_gpu():
    table = _scenario("cuda")
    torch.cuda.synchronize()
    _lib.check_status()
    # an address outside the region is never dereferenced: the row reads as zeros and the status word reports it
    stray = torch.tensor([table.data_ptr() + table.numel() * 4, table.data_ptr() + 2], device="cuda")
    out = embedding_lookup_by_address(stray, 12, table)
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0
    with pytest.raises(Exception):
        _lib.check_status()
    torch.cuda.synchronize()
    _lib.check_status()                                                # cleared by the raise; the context is still usable


@pytest.mark.gpu
def test_pointers_of_the_dynamic_table_round_trip():
    from recsdk_b200.dynamic.hkv import HKVTable

    dev = torch.device("cuda", 0)
    t = HKVTable(8, 1024, dev)
    keys = torch.arange(100, 140, device=dev)
    ptrs, _found = t.find_or_insert_pointers(keys)
    rows = embedding_lookup_by_address(ptrs, 8, t.values_hbm)
    embedding_update_by_address(ptrs, torch.ones(40, 8, device=dev), 0, t.values_hbm)
    again = embedding_lookup_by_address(ptrs, 8, t.values_hbm)
    assert torch.allclose(again, rows + 1)
