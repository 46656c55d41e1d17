"""Sparse convolutions (the layers upstream takes from spconv, swin3d_base.py:915-935, 965-970,
989-994, 1039-1059) against the dense operation restricted to the active sites (the oracle)."""
import pytest
import torch

from oracle import ssw_oracle as O
from tests.cases import make_case, rel_err

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2, torch.float16: 3e-3}


def _scene(dims, batch, n_vox, seed):
    case = make_case(n_vox=n_vox, dims=dims, batch=batch, seed=seed)
    return case["coords"]


@pytest.mark.parametrize("pair_form", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dims,batch,cin,cout", [((9, 10, 11), 2, 6, 16), ((12, 12, 12), 1, 48, 48), ((7, 16, 5), 1, 16, 24)])
def test_submanifold_conv_against_dense(dims, batch, cin, cout, dtype, pair_form, monkeypatch):
    """Both forms of the submanifold convolution: pairs grouped by tap + gather-reduce (sparse
    neighbourhoods) and the dense gathered operand."""
    from sparseswin3d_b200 import sparse_conv, stage

    monkeypatch.setattr(sparse_conv, "PAIR_FORM_MAX_FILL", 1.0 if pair_form else 0.0)
    dev = torch.device("cuda:0")
    coords = _scene(dims, batch, 300, sum(dims))
    g = torch.Generator().manual_seed(cin)
    feats = torch.randn(coords.shape[0], cin, generator=g).to(dtype)
    conv = sparse_conv.SubMConv3d(cin, cout, kernel_size=3, padding=1, bias=True, indice_key="k").to(dev).to(dtype)
    x = stage.SparseVoxels(feats.to(dev), coords.to(dev), dims, batch)
    with torch.no_grad():
        y = conv(x)
        y2 = conv(y.replace_feature(x.features))          # second layer on the same key: rulebook reused
    assert y.indices is x.indices and "k" in x.indice_dict and torch.equal(y.features, y2.features)
    assert (x.indice_dict["k"].seg > 0) == pair_form
    ref = O.subm_conv3d(feats.double(), coords, batch, dims, conv.weight.detach().cpu().double(), conv.bias.detach().cpu().double())
    assert rel_err(y.features.float().cpu(), ref) <= TOL[dtype]
    # the rulebook itself, bit exact: neighbour ids from a dictionary of the coordinates
    lut = {tuple(c): i for i, c in enumerate(coords.tolist())}
    nbr = x.indice_dict["k"].nbr.cpu()
    for i in (0, 17, coords.shape[0] - 1):
        b, z, yy, xx = coords[i].tolist()
        want = [lut.get((b, z + dz, yy + dy, xx + dx), -1) for dz in (-1, 0, 1) for dy in (-1, 0, 1) for dx in (-1, 0, 1)]
        assert nbr[i].tolist() == want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dims,batch,k", [((10, 12, 8), 2, 2), ((9, 11, 7), 1, 2), ((12, 9, 6), 1, 3)])
def test_strided_conv_and_its_inverse_against_dense(dims, batch, k, dtype):
    from sparseswin3d_b200 import sparse_conv, stage

    dev = torch.device("cuda:0")
    coords = _scene(dims, batch, 200, 7 + sum(dims))
    cin, cout = 16, 32
    g = torch.Generator().manual_seed(3)
    feats = torch.randn(coords.shape[0], cin, generator=g).to(dtype)
    down = sparse_conv.SparseConv3d(cin, cout, kernel_size=k, stride=k, bias=False, indice_key="d").to(dev).to(dtype)
    up = sparse_conv.SparseInverseConv3d(cout, cin, kernel_size=k, indice_key="d", bias=False).to(dev).to(dtype)
    x = stage.SparseVoxels(feats.to(dev), coords.to(dev), dims, batch)
    with torch.no_grad():
        y = down(x)
        z = up(y)
    wd, wu = down.weight.detach().cpu().double(), up.weight.detach().cpu().double()
    ref_y, ref_idx, ref_dims = O.strided_conv3d(feats.double(), coords, batch, dims, wd)
    assert list(y.spatial_shape) == ref_dims and y.indices.dtype == torch.int32
    assert torch.equal(y.indices.cpu(), ref_idx)                      # same sites, (b, z, y, x) order
    assert rel_err(y.features.float().cpu(), ref_y) <= TOL[dtype]
    ref_z = O.inverse_conv3d(y.features.double().cpu(), ref_idx, batch, ref_dims, coords, wu)
    assert z.indices is x.indices and list(z.spatial_shape) == list(dims)
    assert rel_err(z.features.float().cpu(), ref_z) <= TOL[dtype]


def test_gradients_flow_through_the_convolutions():
    from sparseswin3d_b200 import sparse_conv, stage

    dev = torch.device("cuda:0")
    dims, batch = (8, 8, 8), 1
    coords = _scene(dims, batch, 120, 5)
    feats = torch.randn(120, 8, device=dev, requires_grad=True)
    net = torch.nn.ModuleList([sparse_conv.SubMConv3d(8, 8, 3, bias=False, indice_key="s"),
                               sparse_conv.SparseConv3d(8, 16, 2, 2, bias=False, indice_key="d"),
                               sparse_conv.SparseInverseConv3d(16, 8, 2, indice_key="d", bias=False)]).to(dev)
    x = stage.SparseVoxels(feats, coords.to(dev), dims, batch)
    for m in net:
        x = m(x)
    x.features.square().sum().backward()
    # against the dense operations differentiated by autograd
    f2 = feats.detach().cpu().double().requires_grad_(True)
    w = [m.weight.detach().cpu().double() for m in net]
    a = O.subm_conv3d(f2, coords, batch, dims, w[0])
    b, bidx, bdims = O.strided_conv3d(a, coords, batch, dims, w[1])
    c = O.inverse_conv3d(b, bidx, batch, bdims, coords, w[2])
    c.square().sum().backward()
    assert rel_err(feats.grad.cpu(), f2.grad) <= 1e-4
    assert all(m.weight.grad is not None for m in net)


def test_patch_merging_and_expand_round_trip_shapes():
    from sparseswin3d_b200 import sparse_conv, stage

    dev = torch.device("cuda:0")
    dims, batch = (14, 14, 14), 2
    coords = _scene(dims, batch, 500, 9)
    x = stage.SparseVoxels(torch.randn(coords.shape[0], 48, device=dev), coords.to(dev), dims, batch)
    pm = sparse_conv.PatchMerging(48, indice_key="pm").to(dev)
    pe = sparse_conv.PatchExpand(96, indice_key="pm").to(dev)
    with torch.no_grad():
        y = pm(x)
        z = pe(y)
    assert y.features.shape[1] == 96 and list(y.spatial_shape) == [7, 7, 7]
    uniq = torch.unique(torch.cat([coords[:, :1], coords[:, 1:] // 2], 1), dim=0)
    assert torch.equal(y.indices.cpu(), uniq.to(torch.int32))         # unique(coords // 2), sorted
    assert z.features.shape == (coords.shape[0], 48) and z.indices is x.indices


def test_full_size_room_properties(monkeypatch):
    """150 000-voxel room, where the dense oracle cannot go: the two forms of the submanifold
    convolution agree with each other, a centre-only kernel is a plain Linear, the rulebook is
    symmetric, and the strided convolution / its inverse conserve what they must."""
    from sparseswin3d_b200 import scenes, sparse_conv, stage

    dev = torch.device("cuda:0")
    coords_np, dims = scenes.room_scene(150_000, seed=0)
    coords = torch.from_numpy(coords_np).to(dev)
    n, C = coords.shape[0], 48
    g = torch.Generator(device=dev).manual_seed(4)
    feats = torch.randn(n, C, device=dev, generator=g)
    conv = sparse_conv.SubMConv3d(C, C, 3, bias=False, indice_key="a").to(dev)
    with torch.no_grad():
        x = stage.SparseVoxels(feats, coords, dims, 1)
        y_pairs = conv(x).features
        assert x.indice_dict["a"].seg > 0                               # the room is sparse: pair form
        monkeypatch.setattr(sparse_conv, "PAIR_FORM_MAX_FILL", 0.0)
        x2 = stage.SparseVoxels(feats, coords, dims, 1)
        y_dense = conv(x2).features
        assert x2.indice_dict["a"].seg == 0
        assert rel_err(y_pairs.cpu(), y_dense.cpu()) <= 1e-5
        # neighbour relation is symmetric: j is i's neighbour through tap t  <=>  i is j's through 26 - t
        nbr = x2.indice_dict["a"].nbr
        i = torch.randint(0, n, (4000,), device=dev, generator=g)
        t = torch.randint(0, 27, (4000,), device=dev, generator=g)
        j = nbr[i, t].long()
        ok = j >= 0
        assert torch.equal(nbr[j[ok], 26 - t[ok]].long(), i[ok])
        assert torch.equal(nbr[:, 13].long(), torch.arange(n, device=dev))   # the centre tap is the voxel itself
        # a kernel with only its centre tap is a Linear over the channels
        w = torch.zeros_like(conv.weight)
        w[13] = conv.weight[13]
        conv.weight.copy_(w)
        assert rel_err(conv(x).features.cpu(), (feats @ w[13]).cpu()) <= 1e-5
        # strided convolution with every tap the identity: each output is the sum of its children;
        # the inverse with every tap the identity hands every child its parent's row
        down = sparse_conv.SparseConv3d(C, C, 2, 2, bias=False, indice_key="d").to(dev)
        up = sparse_conv.SparseInverseConv3d(C, C, 2, indice_key="d", bias=False).to(dev)
        eye = torch.eye(C, device=dev).expand(8, C, C).contiguous()
        down.weight.copy_(eye), up.weight.copy_(eye)
        yd = down(x)
        rb = x.indice_dict["d"]
        has_parent = rb.parent >= 0
        assert rel_err(yd.features.sum(0).cpu(), feats[has_parent].sum(0).cpu()) <= 1e-4
        uniq = torch.unique(torch.cat([coords[has_parent][:, :1], coords[has_parent][:, 1:] // 2], 1), dim=0)
        assert torch.equal(yd.indices.cpu(), uniq.cpu().to(torch.int32))
        z = up(yd)
        want = torch.zeros_like(feats)
        want[has_parent] = yd.features[rb.parent[has_parent].long()]
        assert torch.equal(z.features, want)
