"""How a captured step is wired: the launches of one call are chained with programmatic dependent
launch (a kernel may start while its predecessor drains, and calls griddepcontrol.wait before it
reads anything), and a step forks the second plan's bucketing to a side stream.  The graph a
capture produces must keep (a) programmatic edges only between kernels of this library that
execute griddepcontrol.wait in all their threads before their first read of produced data, and
(b) both predecessors of the second attention call: its own stream's and the side stream's."""
import pytest
import torch

from tests.cases import make_case

pytestmark = pytest.mark.gpu

# every kernel that is launched with the programmatic-serialization attribute waits on its grid
# dependency before its first read: these are the only legal targets of a programmatic edge
WAITING_KERNELS = ("k_reduce", "k_compact", "k_order", "k_scatter", "k_attn_fused", "k_attn_mma", "k_attn_dense",
                   "k_attn_bwd_kv")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_captured_step_keeps_full_join_and_legal_programmatic_edges(dtype):
    from sparseswin3d_b200 import _lib, attention, window

    dev = torch.device("cuda:0")
    case = make_case(n_vox=4000, grid=40, seed=2)
    coords = case["coords"].to(dev)
    qkv = case["qkv"].to(dtype).to(dev)
    table = case["table"].to(dev)
    geoms = [window.resolve_geometry(1, case["dims"], case["window"], s) for s in ((0, 0, 0), (3, 3, 3))]
    pp = attention.plan_params(3, 32, dtype)
    outs = [torch.empty(4000, 96, dtype=dtype, device=dev) for _ in range(2)]
    ref_plans = [window.bucket_windows(coords=coords, geom=g, **pp) for g in geoms]
    scratch = [torch.empty(p.layout.scratch_ints, dtype=torch.int32, device=dev) for p in ref_plans]
    bufs = [torch.empty(p.layout.plan_ints, dtype=torch.int32, device=dev) for p in ref_plans]
    aux = torch.cuda.Stream(device=dev)

    def step():
        cur = torch.cuda.current_stream(dev)
        aux.wait_stream(cur)
        with torch.cuda.stream(aux):
            p1 = window.bucket_windows(coords=coords, geom=geoms[1], scratch=scratch[1], plan_buffer=bufs[1], **pp)
        p0 = window.bucket_windows(coords=coords, geom=geoms[0], scratch=scratch[0], plan_buffer=bufs[0], **pp)
        attention.window_attention_fused(qkv, p0, table, case["scale"], use_mask=False, out=outs[0])
        cur.wait_stream(aux)
        attention.window_attention_fused(qkv, p1, table, case["scale"], use_mask=True, out=outs[1])
        return p0, p1

    want = [attention.window_attention_fused(qkv, ref_plans[i], table, case["scale"], use_mask=bool(i)) for i in range(2)]
    step()
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=dev)
    g = torch.cuda.CUDAGraph(keep_graph=True)
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            plans = step()
    info = _lib.graph_edges(g)
    g.instantiate()
    for o in outs:
        o.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert all(p.stats()["error"] == 0 for p in plans)
    assert torch.equal(outs[0], want[0]) and torch.equal(outs[1], want[1])

    edges = info["edges"]          # (from, to, kind, from_port, to_port), nodes as "<index>:<kernel name>"
    assert info["programmatic"] > 0
    for a, b, kind, _, _ in edges:
        if kind == "programmatic":
            assert any(k in b for k in WAITING_KERNELS), f"programmatic edge into {b}"
    # Two attention calls.  Each starts with k_attn_fused or k_attn_mma; for 16-bit inputs of head_dim
    # 32 the kernel for windows beyond a pack (k_attn_dense) is chained behind k_attn_mma.  The
    # first call has one predecessor, its own plan's last bucketing kernel.  The second has two: the
    # last kernel of the first call (same stream) and the side stream's last bucketing kernel.  A
    # launch that carries the programmatic-serialization attribute turns ALL its kernel
    # predecessors into programmatic edges, the cross-stream one included; what makes that safe is
    # the rule checked above (the target waits for every prerequisite grid before its first read).
    def first_kernel(name):
        return "k_attn_fused" in name or "k_attn_mma" in name

    heads = sorted({e[1] for e in edges if first_kernel(e[1])}, key=lambda n: int(n.split(":")[0]))
    assert len(heads) == 2
    incoming = {n: [e for e in edges if e[1] == n] for n in heads}
    second = [n for n in heads if len(incoming[n]) == 2]
    first = [n for n in heads if len(incoming[n]) == 1]
    assert len(second) == 1 and len(first) == 1
    assert "k_scatter" in incoming[first[0]][0][0]
    assert sum("k_scatter" in e[0] for e in incoming[second[0]]) == 1      # the join with the side stream
    assert sum("k_attn" in e[0] for e in incoming[second[0]]) == 1         # and the stream's own order
    for n in {e[1] for e in edges if "k_attn_dense" in e[1]}:               # chained behind its k_attn_mma
        inc = [e for e in edges if e[1] == n]
        assert len(inc) == 1 and "k_attn_mma" in inc[0][0]
    # nothing but kernels of one call's chain and memsets in front of them: the first kernel of a
    # chain is an ordinary launch, fully ordered behind the clears
    for a, b, kind, _, _ in edges:
        if "k_count" in b:
            assert kind == "full"
