"""Gradients of the fused attention (recomputing backward kernels) against the unfused operator
chain, whose own backward operators are pinned to upstream's by tests/test_coo_ops_gpu.py."""
import pytest
import torch

from tests.cases import make_case, rel_err

pytestmark = pytest.mark.gpu


def _module_and_input(case, dev, seed=0):
    from sparseswin3d_b200.attention import WindowAttentionSparse
    from sparseswin3d_b200.voxels import WindowedVoxels

    C = case["heads"] * case["head_dim"]
    torch.manual_seed(seed)
    m = WindowAttentionSparse(C, case["heads"], case["window"], qkv_bias=True).to(dev)
    torch.nn.init.normal_(m.relative_position_bias_table, std=0.5)
    feats = torch.randn(case["coords"].shape[0], C, device=dev)
    make_x = lambda f: WindowedVoxels(f, case["indices"].to(dev), case["n_windows"], (case["n"],))
    return m, feats, make_x


def _grads(m, feats, make_x, mask, fused, weight):
    f = feats.detach().clone().requires_grad_(True)
    m.zero_grad(set_to_none=True)
    out = m(make_x(f), mask, fused=fused).features
    (out * weight).sum().backward()
    return (out.detach(), f.grad.detach().clone(), m.relative_position_bias_table.grad.detach().clone(),
            m.qkv.weight.grad.detach().clone())


@pytest.mark.parametrize("n_vox,grid,heads,hd,shift", [
    (400, 16, 3, 32, (3, 3, 3)),    # small windows, shifted and masked
    (600, 14, 2, 16, (0, 0, 0)),    # windows above one tile (c up to ~100): the large-window items
    (900, 12, 6, 16, (3, 3, 3)),    # dense-ish, many heads
    (700, 18, 6, 16, (4, 4, 4)),    # window 9: the bias table (17^3 x 6) is too large for the shared-memory copy
    (800, 14, 6, 32, (3, 3, 3)),    # C = 192: the pack kernel holds its pair arrays for a part of the heads at a time
    (300, 40, 3, 32, (0, 0, 0)),    # windows of one or two voxels: packs of many windows
])
def test_fused_backward_matches_unfused_chain(n_vox, grid, heads, hd, shift):
    dev = torch.device("cuda:0")
    window = (9, 9, 9) if shift == (4, 4, 4) else (7, 7, 7)
    case = make_case(n_vox=n_vox, grid=grid, heads=heads, head_dim=hd, shift=shift, seed=n_vox, window=window)
    m, feats, make_x = _module_and_input(case, dev)
    mask = case["mask"].to(dev) if case["mask"] is not None else None
    weight = torch.randn(n_vox, heads * hd, device=dev)
    o_u, gf_u, gt_u, gw_u = _grads(m, feats, make_x, mask, False, weight)
    o_f, gf_f, gt_f, gw_f = _grads(m, feats, make_x, mask, True, weight)
    assert rel_err(o_f.cpu(), o_u.cpu()) <= 2e-5
    assert rel_err(gf_f.cpu(), gf_u.cpu()) <= 1e-4      # d features (through dqkv and the qkv Linear)
    assert rel_err(gw_f.cpu(), gw_u.cpu()) <= 1e-4      # d qkv weight
    assert rel_err(gt_f.cpu(), gt_u.cpu()) <= 1e-4      # d bias table (scatter-add over all pairs)


def test_fused_backward_bf16_padded_plan():
    """16-bit tensors use the padded plan; the backward reads the same work list."""
    from sparseswin3d_b200 import attention, window

    dev = torch.device("cuda:0")
    case = make_case(n_vox=1500, grid=24, heads=3, head_dim=32, shift=(3, 3, 3), seed=5)
    geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    qkv32 = case["qkv"].to(dev)
    table = case["table"].to(dev)
    go = torch.randn(1500, 96, device=dev)
    plan32 = window.bucket_windows(coords=case["coords"].to(dev), geom=geom, **attention.plan_params(3, 32, torch.float32))
    plan16 = window.bucket_windows(coords=case["coords"].to(dev), geom=geom, **attention.plan_params(3, 32, torch.bfloat16))
    assert plan16.layout.padded == 1
    q16 = qkv32.bfloat16()
    d32, t32 = attention.window_attention_fused_backward(q16.float(), go.bfloat16().float(), plan32, table, case["scale"], True)
    d16, t16 = attention.window_attention_fused_backward(q16, go.bfloat16(), plan16, table, case["scale"], True)
    assert d16.dtype == torch.bfloat16
    assert rel_err(d16.float().cpu(), d32.cpu()) <= 2e-2   # output rounding of the 16-bit gradient rows
    assert rel_err(t16.cpu(), t32.cpu()) <= 1e-4           # the table gradient is accumulated in fp32 either way
