"""Host-side logic that needs no GPU: edge-index helpers, global-token helpers, module plumbing."""
import numpy as np
import pytest
import torch

from helpers import load_golden
from oracle import edge_layout_oracle as elo
from oracle import sparse_attn_oracle as sao


@pytest.fixture()
def sp_state():
    import torchgt_b200.gt_sp.initialize as init
    init.destroy_sequence_parallel()
    yield init
    init.destroy_sequence_parallel()


def _fake_group(init, world, rank=0):
    init._state.group, init._state.world_size, init._state.rank = object(), world, rank
    init.set_global_token_num(1)


def test_edge_helpers_are_bit_exact_with_the_reference():
    from torchgt_b200.gt_sp import utils
    g = load_golden("edges.npz")
    t = lambda a: torch.from_numpy(a)
    assert torch.equal(utils.fix_edge_index(t(g["ring"]), 4), t(g["ring_fixed"]))
    assert torch.equal(utils.adjust_edge_index_nomerge(t(g["ring_fixed"]), 2), t(g["ring_adjusted_L2"]))
    assert torch.equal(utils.flatten_edge_index_nopad([t(g["ring_adjusted_L2"]), t(g["ring_adjusted_L2"])[:, :3]], 6),
                       t(g["ring_flat_6"]))
    for i in range(4):
        n, sub = int(g[f"rand{i}_n"]), int(g[f"rand{i}_sub"])
        fixed = utils.fix_edge_index(t(g[f"rand{i}_in"]), n)
        assert torch.equal(fixed, t(g[f"rand{i}_fixed"]))
        assert torch.equal(utils.adjust_edge_index_nomerge(fixed, sub), t(g[f"rand{i}_adjusted"]))
    assert torch.equal(utils.flatten_edge_index_nopad([t(g["flat_in0"]), t(g["flat_in1"]), t(g["flat_in2"])], 10),
                       t(g["flat_out_10"]))
    # integer arithmetic agrees with the reference's float32 floor wherever that is exact
    big = torch.arange(0, 2 ** 24, 4099).view(1, -1).repeat(2, 1)
    for sub in (1, 7, 64000, 108751):
        assert np.array_equal(utils.adjust_edge_index_nomerge(big, sub).numpy(),
                              elo.adjust_edge_index_nomerge(big.numpy(), sub))


def test_global_token_helpers(sp_state):
    from torchgt_b200.gt_sp import utils
    world, L = 4, 3
    _fake_group(sp_state, world)
    rows = list(range(0, world * (L + 1), L + 1))
    sp_state.set_global_token_indices(rows)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(2, world * (L + 1), 5, generator=gen)
    body = [i for i in range(x.size(1)) if i not in rows]
    mean = x[:, rows].mean(dim=1, keepdim=True)
    assert torch.allclose(utils.merge_global_token(x, 1), torch.cat([x[:, body], mean], dim=1))
    assert torch.allclose(utils.merge_global_token0(x, 1), torch.cat([mean, x[:, body]], dim=1))
    merged0 = utils.merge_global_token0(x, 1)                       # [2, 1 + 12, 5]
    ext0 = utils.extend_global_token0(merged0, 1)
    assert ext0.shape == x.shape
    for r in range(world):
        assert torch.equal(ext0[:, r * (L + 1)], merged0[:, 0])
        assert torch.equal(ext0[:, r * (L + 1) + 1:(r + 1) * (L + 1)], merged0[:, 1 + r * L:1 + (r + 1) * L])
    y = utils.copy_global_token0(x.clone(), 1)
    for r in rows:
        assert torch.equal(y[:, r], x[:, 0])
    assert torch.equal(y[:, body], x[:, body])
    chunks = utils.split_tensor_along_second_dim(x, world, contiguous_split_chunks=True)
    assert len(chunks) == world and all(c.is_contiguous() and c.shape[1] == L + 1 for c in chunks)
    # last-batch indices are used when the flag is set
    sp_state.set_last_batch_global_token_indices([0, 2, 4, 6])
    sp_state.last_batch_flag(True)
    y = utils.copy_global_token0(x[:, :8].clone(), 1)
    assert torch.equal(y[:, 2], x[:, 0]) and torch.equal(y[:, 3], x[:, 3])


def test_core_attention_attributes_and_sequence_parallel_head_split(sp_state):
    from torchgt_b200 import CoreAttention
    core = CoreAttention(64, 0.5, 8, 1)
    assert (core.hidden_size_per_attention_head, core.num_attention_heads_per_partition, core.num_heads) == (8, 8, 8)
    assert core.attention_dropout_rate == 0.5 and isinstance(core.att_dropout, torch.nn.Dropout)
    assert list(core.parameters()) == [] and list(core.buffers()) == []
    _fake_group(sp_state, 4)
    core = CoreAttention(64, 0.5, 8)
    assert core.num_attention_heads_per_partition == 2 and core.hidden_size_per_partition == 16


def test_dense_bias_lookup_matches_the_reference_indexing():
    from torchgt_b200.attn_module import edge_bias_from_dense
    gen = torch.Generator().manual_seed(1)
    b, h, n = 2, 4, 9
    ei = torch.randint(0, b * n, (2, 40), generator=gen)
    ei[1] = (ei[0] // n) * n + ei[1] % n          # edges stay inside their graph
    dense = torch.randn(b, h, n, n, generator=gen)
    # the reference: permute(0,2,3,1).unsqueeze(2).repeat(1,1,b,1,1).view(b*n, b*n, h)[src, dst]
    ref = dense.permute(0, 2, 3, 1).contiguous().unsqueeze(2).repeat(1, 1, b, 1, 1).view(b * n, b * n, h)[ei[0], ei[1]]
    assert torch.equal(edge_bias_from_dense(dense, ei, b, n, h), ref)
    single = dense[:1]
    ei1 = ei % n
    assert torch.equal(edge_bias_from_dense(single, ei1, 1, n, h), sao.dense_bias_to_edges(single, ei1))
    node_level = torch.randn(1, n, n, h, generator=gen)           # [b, N, N, heads] form
    assert torch.equal(edge_bias_from_dense(node_level, ei1, 1, n, h), node_level[0][ei1[0], ei1[1]])
    with pytest.raises(ValueError):
        edge_bias_from_dense(torch.zeros(1, h, n + 1, n + 1), ei1, 1, n, h)
    # heads == nodes: the shape fits both forms; it is never guessed, the caller names the form
    square = torch.randn(1, n, n, n, generator=gen)
    with pytest.raises(ValueError, match="fits both"):
        edge_bias_from_dense(square, ei1, 1, n, n)
    assert torch.equal(edge_bias_from_dense(square, ei1, 1, n, n, "node"), square[0][ei1[0], ei1[1]])
    assert torch.equal(edge_bias_from_dense(square, ei1, 1, n, n, "graph"), square[0][:, ei1[0], ei1[1]].t())


def test_the_op_refuses_host_tensors():
    """There is no CPU path: a call with host tensors must fail loudly, not fall back."""
    from torchgt_b200 import CoreAttention, SparseGraph, sparse_graph_attention
    q = torch.randn(5, 2, 8)
    ei = torch.tensor([[0, 1], [1, 2]])
    with pytest.raises(RuntimeError, match="CUDA"):
        sparse_graph_attention(q, q, q, ei)
    with pytest.raises(RuntimeError, match="CUDA"):
        SparseGraph(ei, 5)
    with pytest.raises(RuntimeError, match="CUDA"):
        CoreAttention(16, 0.0, 2)(q[None], q[None], q[None], None, ei, "sparse")
    with pytest.raises(NotImplementedError):
        CoreAttention(16, 0.0, 2)(q[None], q[None], q[None], None, ei, "full")


def test_product_code_never_imports_the_oracle():
    import pathlib
    pkg = pathlib.Path(__file__).resolve().parent.parent / "torchgt_b200"
    for path in pkg.rglob("*.py"):
        text = path.read_text()
        assert "import oracle" not in text and "from oracle" not in text, path


def test_graphormer_shell_loads_reference_checkpoints_and_counts_the_same_parameters(sp_state):
    from torchgt_b200.graphormer import Graphormer
    g = load_golden("graphormer_node_level.npz")
    model = Graphormer(3, 8, 24, 64, 7, 1, 0.0, 0.0, 0.0, 64, 1)
    state = {k[len("param/"):]: torch.from_numpy(v) for k, v in g.items() if k.startswith("param/")}
    assert sorted(state) == sorted(model.state_dict())          # same keys as the reference's state_dict
    model.load_state_dict(state, strict=True)
    readme_model = Graphormer(4, 8, 128, 64, 40, 1, 0.3, 0.1, 0.5, 64, 1)
    n = sum(p.numel() for p in readme_model.parameters())
    assert n == 111913 == int(g["params_of_the_readme_model"])   # the count the reference's README logs


def test_gt_and_graph_level_shells_load_reference_checkpoints(sp_state):
    from torchgt_b200.graphormer import GraphormerGraphLevel
    from torchgt_b200.gt import GTGraphLevel, GTNodeLevel
    graph_level = (2, 8, 64, 0.0, 0.0, 64, "ZINC", "multi_hop", 5, 0.0, 5)
    for model, name in ((GTNodeLevel(3, 8, 20, 64, 6, 1, 0.0, 0.0, 0.0, 64, 0), "gt_node_level.npz"),
                        (GTGraphLevel(*graph_level), "gt_graph_level.npz"),
                        (GraphormerGraphLevel(*graph_level), "graphormer_graph_level.npz")):
        g = load_golden(name)
        state = {k[len("param/"):]: torch.from_numpy(v) for k, v in g.items() if k.startswith("param/")}
        assert set(state) == set(model.state_dict())
        model.load_state_dict(state, strict=True)


def test_layer_norm_and_linear_modules_are_torch_modules_on_the_cpu():
    """On host tensors (and for shapes the kernels do not cover) the two dense modules of the model shells
    are ``nn.LayerNorm`` / ``nn.Linear`` themselves: same parameters, same ``state_dict`` keys, same numbers."""
    from torchgt_b200.layer_norm import LayerNorm
    from torchgt_b200.linear import Linear
    torch.manual_seed(5)
    ln, ref_ln = LayerNorm(64), torch.nn.LayerNorm(64)
    lin, ref_lin = Linear(64, 64), torch.nn.Linear(64, 64)
    assert list(ln.state_dict()) == list(ref_ln.state_dict()) and list(lin.state_dict()) == list(ref_lin.state_dict())
    assert isinstance(ln, torch.nn.LayerNorm) and isinstance(lin, torch.nn.Linear)
    ref_ln.load_state_dict(ln.state_dict())
    ref_lin.load_state_dict(lin.state_dict())
    x = torch.randn(7, 64, requires_grad=True)
    y = lin(ln(x))
    y.sum().backward()
    x2 = x.detach().clone().requires_grad_()
    y2 = ref_lin(ref_ln(x2))
    y2.sum().backward()
    assert torch.equal(y, y2) and torch.equal(x.grad, x2.grad)
    assert torch.equal(lin.weight.grad, ref_lin.weight.grad) and torch.equal(ln.weight.grad, ref_ln.weight.grad)
