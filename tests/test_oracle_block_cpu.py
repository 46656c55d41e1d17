"""CPU: the oracle's Swin block (dense per-window attention inside LayerNorm / Linear / GELU /
residuals) against the same block assembled from the oracle's COO operator chain - the restatement
that the upstream fixtures pin (tests/test_oracle_golden.py)."""
import torch
import torch.nn.functional as F

from oracle import ssw_oracle as O
from tests.cases import make_case, rel_err


def test_block_restatement_agrees_with_operator_chain():
    dims, win, shift, H, C = (12, 16, 14), (7, 7, 7), (3, 3, 3), 3, 48
    case = make_case(n_vox=400, dims=dims, window=win, shift=shift, heads=H, head_dim=C // H, seed=2)
    g = torch.Generator().manual_seed(1)
    r = lambda *s: torch.randn(*s, generator=g)
    prm = {"norm1.weight": 1 + 0.2 * r(C), "norm1.bias": 0.1 * r(C), "attn.qkv.weight": r(3 * C, C) * C ** -0.5,
           "attn.qkv.bias": 0.1 * r(3 * C), "attn.relative_position_bias_table": 0.5 * r(13 ** 3, H),
           "attn.proj.weight": r(C, C) * C ** -0.5, "attn.proj.bias": 0.1 * r(C), "norm2.weight": 1 + 0.2 * r(C),
           "norm2.bias": 0.1 * r(C), "mlp.linear1.weight": r(4 * C, C) * C ** -0.5, "mlp.linear1.bias": 0.1 * r(4 * C),
           "mlp.linear2.weight": r(C, 4 * C) * (4 * C) ** -0.5, "mlp.linear2.bias": 0.1 * r(C)}
    feats = r(400, C)
    got = O.swin_block(feats, case["coords"], 1, dims, win, shift, prm, H)
    # the same block, attention through the operator chain on upstream's (indices, mask) interface
    x = feats.double()
    d = {k: v.double() for k, v in prm.items()}
    h = F.layer_norm(x, (C,), d["norm1.weight"], d["norm1.bias"], 1e-5)
    a = O.window_attention_forward(h, case["indices"], case["n_windows"], case["n"], H, d["attn.qkv.weight"], d["attn.qkv.bias"],
                                   d["attn.proj.weight"], d["attn.proj.bias"], d["attn.relative_position_bias_table"],
                                   case["rpi"], case["mask"])[0]
    x = x + a
    h = F.layer_norm(x, (C,), d["norm2.weight"], d["norm2.bias"], 1e-5)
    want = x + F.linear(F.gelu(F.linear(h, d["mlp.linear1.weight"], d["mlp.linear1.bias"])), d["mlp.linear2.weight"],
                        d["mlp.linear2.bias"])
    assert rel_err(got, want) <= 1e-6   # the operator chain keeps some fp32 intermediates
    # depth 2 = W-MSA block then SW-MSA block
    two = O.basic_layer(feats, case["coords"], 1, dims, win, [prm, prm], H)
    step = O.swin_block(O.swin_block(feats, case["coords"], 1, dims, win, (0, 0, 0), prm, H), case["coords"], 1, dims, win, shift, prm, H)
    assert torch.equal(two, step)
