"""Shared helpers of the test-suite: error metrics, seeded graphs, golden loading."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"

# Tolerances of the parity contract: fp32 results within 1e-5, bf16 within 1e-2, both measured as
# max |x - ref| relative to max |ref| of the tensor.
TOL_F32 = 1e-5
TOL_BF16 = 1e-2


def rel_err(x, ref) -> float:
    x = np.asarray(x.detach().double().cpu() if isinstance(x, torch.Tensor) else x, dtype=np.float64)
    ref = np.asarray(ref.detach().double().cpu() if isinstance(ref, torch.Tensor) else ref, dtype=np.float64)
    assert x.shape == ref.shape, (x.shape, ref.shape)
    denom = max(float(np.abs(ref).max()) if ref.size else 0.0, 1e-30)
    return float(np.abs(x - ref).max() / denom) if ref.size else 0.0


def load_golden(name: str):
    with np.load(GOLDEN / name) as z:
        return {k: z[k] for k in z.files}


def random_graph(seed: int, n: int, avg_in_degree: float, hub: bool = True, duplicates: bool = True,
                 empty_rows: bool = True) -> torch.Tensor:
    """[2, E] int64 edges: random in-edges + self loops (+ a hub row 0 linked to and from all rows)."""
    gen = torch.Generator().manual_seed(seed)
    e = int(n * avg_in_degree)
    parts = [torch.stack([torch.randint(0, n, (e,), generator=gen), torch.randint(0, n, (e,), generator=gen)])]
    loops = torch.arange(n)
    parts.append(torch.stack([loops, loops]))
    if hub and n > 1:
        others = torch.arange(1, n)
        zeros = torch.zeros(n - 1, dtype=torch.long)
        parts += [torch.stack([others, zeros]), torch.stack([zeros, others])]
    ei = torch.cat(parts, dim=1)
    if not duplicates:
        ei = torch.unique(ei, dim=1)
    ei = ei[:, torch.randperm(ei.shape[1], generator=gen)]
    if empty_rows:
        ei = ei[:, ei[1] % 7 != 3]
    return ei.contiguous()


def clustered_graph(seed: int, n_nodes: int, n_clusters: int, cluster_edges: int, cross_fraction: float):
    """Synthetic stand-in for the reordered 64K-node benchmark batch: global node 0, ``n_nodes`` nodes in
    ``n_clusters`` equal clusters, self loops, global-token edges both ways, and ``cluster_edges`` random
    edges of which ``cross_fraction`` cross clusters.  Returns ([2, E] int64, n_rows = n_nodes + 1)."""
    gen = torch.Generator().manual_seed(seed)
    size = n_nodes // n_clusters
    nodes = torch.arange(1, n_nodes + 1)
    zeros = torch.zeros(n_nodes, dtype=torch.long)
    src = torch.randint(0, n_nodes, (cluster_edges,), generator=gen)
    cross = torch.rand(cluster_edges, generator=gen) < cross_fraction
    same = (src // size) * size + torch.randint(0, size, (cluster_edges,), generator=gen)
    anywhere = torch.randint(0, n_nodes, (cluster_edges,), generator=gen)
    dst = torch.where(cross, anywhere, same)
    ei = torch.cat([torch.stack([nodes, nodes]), torch.stack([nodes, zeros]), torch.stack([zeros, nodes]),
                    torch.stack([src + 1, dst + 1])], dim=1)
    return ei.contiguous(), n_nodes + 1
