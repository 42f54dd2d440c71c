#!/usr/bin/env python
"""Benchmark of the sparse graph-attention hot path (forward + backward) in edges/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--dtype fp32|bf16]

One *step* is one forward+backward of the attention over one synthetic batch; one *edge* is one
(source, destination) pair evaluated for all 8 heads of the model.

N = 1   The 64K-node micro-benchmark batch (64,001 rows, 526,450 edges, 8 heads x 8, fp32, scalar edge
        bias).  ``value`` times the C-ABI calls (captured once in a CUDA graph, inputs resident in HBM,
        four rotating input sets so no step finds its inputs in L2); ``e2e`` goes through the public
        Python API from pinned host buffers (uploads of q, k, v, bias, dO and the edge list, layout
        build, forward, backward, download of out, dq, dk, dv, dbias — every step).
N > 1   One process per GPU under torchrun.  Weak scaling of the Ulysses layer: every rank owns 64,000
        nodes of an N x 64,000-node graph and all 8 heads outside attention; the step is
        DistributedAttentionNoMerge forward+backward (all-to-all, attention over all rows with 8/N heads,
        all-to-all back, and the reverse in backward).  value = N x 526,450 edges / max-over-ranks time.

``--impl reference`` times the reference's own CPU implementation of the path (its PyTorch operation
sequence restated in oracle/, all host threads) on the same workload, rank 0 only.

Further legs of the default run: ``more_workloads`` (64K bf16, 870K fp32 / bf16; ``TGT_BENCH_MORE=0`` skips),
``epoch`` (the reference's training epoch; ``TGT_BENCH_EPOCH=0`` skips it and, at N > 1, the
``weak_scaling_training_step`` leg), at N > 1 also the parity self-check, ``attention_only``, ``exchange_only``.
``TGT_BENCH_KERNEL_LIST=1`` (N > 1) adds the device time of every kernel of the replayed step on rank 0;
``--workload 870k`` (N = 1) makes the long-sequence batch the headline; ``--profile`` keeps the run short for
profilers.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HEADS, HEAD_DIM = 8, 8
NODES_PER_RANK = 64000
ROTATING_SETS = 4


def ncu_traffic(workload, dtype_name):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of each phase, as recorded next to the ncu
    summary of that workload under profiles/ (the dQ phase includes the row-statistics kernel); None when
    no capture of this workload is on file."""
    path = ROOT / "profiles" / f"sparse_attn_{workload}_{dtype_name}_traffic.json"
    try:
        return {k: float(v) for k, v in json.loads(path.read_text())["dram_bytes_per_launch"].items()}
    except Exception:
        return None


def measured_hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def algorithmic_bytes(n_rows, n_edges, heads, head_dim, elem, bias_bytes):
    """Bytes the op must move: Q read + per-edge K/V/bias gathers + output write, and the matching
    terms of the two backward passes.  Indices and row statistics are not counted."""
    r = heads * head_dim * elem
    fwd = 2 * n_rows * r + n_edges * (2 * r + bias_bytes)
    dq = 4 * n_rows * r + n_edges * (2 * r + bias_bytes)
    dkv = 4 * n_rows * r + n_edges * (2 * r + bias_bytes)
    return {"fwd_kernel": fwd, "bwd_dq_kernel": dq, "bwd_dkv_kernel": dkv}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


# ---------------------------------------------------------------------------------------------------
def make_inputs(n_rows, n_edges, dtype, seed, device):
    gen = torch.Generator().manual_seed(seed)
    q, k, v, dout = (torch.randn(n_rows, HEADS, HEAD_DIM, generator=gen) for _ in range(4))
    bias = torch.randn(n_edges, generator=gen) * 0.1
    cast = lambda t: t.to(dtype).to(device) if device is not None else t.to(dtype)
    return cast(q), cast(k), cast(v), cast(dout), (bias.to(device) if device is not None else bias)


def cpu_reference_rate(edge_index, n_rows, steps, warmup, time_limit_s=20.0, seed=1234, with_bias=True):
    """Edges/s of the reference's CPU operation sequence (oracle/sparse_attn_oracle.sparse_attention_ops,
    float32, autograd backward) with all host threads, on a bounded edge sample of the workload."""
    from oracle.sparse_attn_oracle import sparse_attention_ops
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    q, k, v, dout, bias = make_inputs(n_rows, edge_index.shape[1], torch.float32, seed, None)

    def one(ei, b):
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        t0 = time.perf_counter()
        out = sparse_attention_ops(qq, kk, vv, ei, b if with_bias else None)
        out.backward(dout)
        return time.perf_counter() - t0

    n_edges = edge_index.shape[1]
    probe_edges = min(n_edges, 65536)
    probe = edge_index[:, torch.randperm(n_edges, generator=torch.Generator().manual_seed(1))[:probe_edges]]
    one(probe, bias[:probe_edges])
    t_probe = one(probe, bias[:probe_edges])
    per_edge = t_probe / probe_edges
    sample_edges = int(min(n_edges, max(probe_edges, time_limit_s / max(steps + warmup, 1) / per_edge)))
    if sample_edges >= n_edges:
        ei, b, what = edge_index, bias, f"full workload ({n_edges} edges, {n_rows} rows)"
    else:
        sel = torch.randperm(n_edges, generator=torch.Generator().manual_seed(2))[:sample_edges]
        ei, b = edge_index[:, sel].contiguous(), bias[sel].contiguous()
        what = f"random sample of {sample_edges} of {n_edges} edges over all {n_rows} rows"
    for _ in range(warmup):
        one(ei, b)
    times = [one(ei, b) for _ in range(steps)]
    mean = sum(times) / len(times)
    return {"value": ei.shape[1] / mean, "unit": "edges/s", "cores": cores, "kind": "port",
            "sample": f"{what}; {warmup} warm-up + {steps} timed fwd+bwd, mean {mean * 1e3:.1f} ms"}, mean


def run_reference_arm(args, rank):
    if rank != 0:
        return
    edge_index, n_rows = load_workload(args.workload, ranks=args.gpus)
    if args.gpus > 1:   # the row numbering of the sequence-parallel layer (one global-token slot per rank)
        from torchgt_b200.gt_sp.utils import adjust_edge_index_nomerge
        edge_index = adjust_edge_index_nomerge(edge_index, NODES_PER_RANK)
        n_rows = args.gpus * (NODES_PER_RANK + 1)
    # N = 1 times the op with a scalar edge bias (gradient included), N > 1 the layer's own call: no bias
    base, mean = cpu_reference_rate(edge_index, n_rows, args.steps, max(args.warmup, 1), time_limit_s=150.0,
                                    with_bias=args.gpus == 1)
    line = {
        "impl": "reference", "metric": "sparse_graph_attention_fwd_bwd_edges_per_s", "value": base["value"],
        "unit": "edges/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": mean * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus, n_rows, edge_index.shape[1], "fp32", args.workload),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


WORKLOADS = {
    "64k": "sparse-attention op microbench: 64,000 nodes per GPU + global node, 8 clusters of 8,000 per GPU, "
           "17.5% of edges crossing clusters, scalar edge bias, fwd+bwd",
    "870k": "long-sequence batch: 870,000 nodes + global node, 18,214,272 edges, power-law out-degrees "
            "(exponent 2.1), 8 clusters with 7.1% of edges cut, scalar edge bias, fwd+bwd",
}


def load_workload(name, ranks=1):
    from torchgt_b200.synthetic import benchmark_64k, benchmark_870k
    if name == "870k":
        if ranks != 1:
            raise SystemExit("--workload 870k is a single-GPU workload")
        return benchmark_870k()
    return benchmark_64k(ranks=ranks)


def workload_config(n_gpus, n_rows, n_edges, dtype, name="64k"):
    return {"workload": WORKLOADS[name],
            "rows": n_rows, "edges": n_edges, "heads": HEADS, "head_dim": HEAD_DIM, "io_dtype": dtype,
            "parallelism": "single GPU" if n_gpus == 1 else f"Ulysses sequence parallel x{n_gpus} (heads sharded)",
            "l2": f"{ROTATING_SETS} rotating input sets, footprint > 126 MB L2, no explicit flush"}


# ---------------------------------------------------------------------------------------------------
EPOCH_SHAPES = {
    # (seed, nodes, random edges, cross-cluster fraction, zipf exponent) per batch; features; classes
    "64k": {"batches": ((42, 64000, 334450, 0.315, 0.0), (43, 37608, 228357 - 3 * 37608, 0.315, 0.0)),
            "features": 128, "classes": 40, "epochs": 12},
    # the shape of the reference's ogbn-products run at sequence length 870,000: a full batch and a shorter
    # last one (about 599 K nodes and 9.2 M edges; 8 clusters of 74,878 nodes here)
    "870k": {"batches": ((42, 870000, 18214272 - 3 * 870000, 0.0812, 2.1),
                         (43, 599024, 9200000 - 3 * 599024, 0.0812, 2.1)),
             "features": 100, "classes": 47, "epochs": 8},
}


def epoch_benchmark(rank, world, dev, workload="64k"):
    """End-to-end training epoch of the node-level Graphormer at sequence length 64K or 870K, timed the
    way the reference times it (main_sp_sparse_node_level.py:196-221): per iteration from "inputs are on
    the GPU" to "optimizer step done and device idle", summed over the epoch's two batches (64,000 and
    37,608 nodes, the sizes of its ogbn-arxiv run; 870,000 and 599,024 nodes with 18.2 M and 9.2 M edges
    for the ogbn-products shape), averaged over the epochs after the fourth.  The sequence
    is split over the ranks (strong scaling, as in the reference); weights are replicated and their
    gradients averaged with one flat all-reduce."""
    import torch.distributed as dist
    from torch.nn import functional as F
    from torchgt_b200 import SparseGraph
    from torchgt_b200.graphormer import Graphormer
    from torchgt_b200.gt_sp import initialize as sp
    from torchgt_b200.gt_sp.reducer import Reducer
    from torchgt_b200.gt_sp.utils import adjust_edge_index_nomerge
    from torchgt_b200.synthetic import clustered_edges
    torch.manual_seed(42)
    # the dense layers around the path are library GEMMs; TF32 is what the reference's PyTorch (1.10) used
    # for them by default on Ampere-class GPUs
    torch.backends.cuda.matmul.allow_tf32 = True
    shape = EPOCH_SHAPES[workload]
    epochs, n_feat, n_cls = shape["epochs"], shape["features"], shape["classes"]
    model = Graphormer(4, 8, n_feat, 64, n_cls, 1, 0.3, 0.1, 0.5, 64, 1).to(dev).train()
    if world > 1:
        for p in model.parameters():
            dist.broadcast(p.data, src=0)
    opt = torch.optim.AdamW(model.parameters(), lr=2e-4, weight_decay=0.01, fused=True, capturable=True)
    batches = []
    for seed, n_nodes, random_edges, cross, zipf in shape["batches"]:
        ei, n_rows = clustered_edges(seed, n_nodes, 8, random_edges, cross, zipf_exponent=zipf)
        L = n_nodes // world
        gen = torch.Generator().manual_seed(seed + 100)
        x = torch.randn(n_nodes, n_feat, generator=gen)
        y = torch.randint(0, n_cls, (n_nodes,), generator=gen)
        ei = adjust_edge_index_nomerge(ei, L) if world > 1 else ei
        graph = SparseGraph(ei.to(dev), world * (L + 1) if world > 1 else n_rows)
        graph.by_src
        rows = list(range(0, world * (L + 1), L + 1))
        batches.append((x[rank * L:(rank + 1) * L].to(dev), y[rank * L:(rank + 1) * L].to(dev), graph, rows,
                        n_nodes, ei.shape[1]))
    params = [p for p in model.parameters()]
    reducer = Reducer().init(model) if world > 1 else None

    def iteration(x, y, graph, rows):
        if world > 1:
            sp.set_global_token_indices(rows)
        out = model(x, None, graph, attn_type="sparse")
        loss = F.nll_loss(out, y)
        if reducer is not None:
            reducer.prepare()                   # gradients accumulate straight into one flat buffer
            loss.backward()                     # its all-reduce starts when the last gradient has arrived
            reducer.synchronize()
        else:
            opt.zero_grad(set_to_none=True)
            loss.backward()
        opt.step()
        return loss

    def run_epochs(step_fns):
        epoch_times, losses = [], []
        for epoch in range(1, epochs + 1):
            t_epoch = 0.0
            for fn in step_fns:
                torch.cuda.synchronize()
                t1 = time.perf_counter()
                loss = fn()
                torch.cuda.synchronize()
                t_epoch += time.perf_counter() - t1
            losses.append(float(loss.detach()))
            if epoch > 4:
                epoch_times.append(t_epoch)
        t = torch.tensor([sum(epoch_times) / len(epoch_times)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), losses

    eager_time, losses = run_epochs([lambda b=b: iteration(b[0], b[1], b[2], b[3]) for b in batches])
    result = {"epoch_time_s": eager_time, "eager_epoch_time_s": eager_time, "timing": "eager PyTorch step",
              "iterations_per_epoch": len(batches),
              "batches": [{"nodes": b[4], "edges": b[5]} for b in batches],
              "model": f"Graphormer node-level, 4 layers, hidden 64, 8 heads, ffn 64, {n_feat} features -> {n_cls} "
                       f"classes, {sum(p.numel() for p in params):,} parameters, dropout as the reference's defaults",
              "includes": "forward, nll_loss, backward, flat gradient all-reduce (N > 1), fused AdamW step; inputs and "
                          "edge layouts resident on the GPU, as the reference times it",
              "dense_layers": "forward products and input gradients are library GEMMs (TF32), dropout, GELU, loss and "
                              "optimizer are torch's; LayerNorm (both directions) and the weight / bias gradients of "
                              "the 64-wide linear layers are this library's kernels (csrc/layer_norm.cu, "
                              "csrc/linear_wgrad.cu): at 64 columns over 64,000 rows torch's own took 3.8 ms and 2.4 "
                              "ms of a 8.0 ms iteration; the attention kernels are about 0.55 ms of the 2.7 ms left",
              "sequence_parallel": world, "first_loss": losses[0], "last_loss": losses[-1]}
    if os.environ.get("TGT_BENCH_EPOCH_GRAPH", "1") != "0":
        # the same iteration (forward, loss, backward, gradient all-reduce, optimizer step) captured once per
        # batch in a CUDA graph: the step is launch-bound when issued kernel by kernel from Python
        graphs, static_loss = [], []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        for b in batches:
            with torch.cuda.stream(side):
                iteration(b[0], b[1], b[2], b[3])
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                static_loss.append(iteration(b[0], b[1], b[2], b[3]))
            graphs.append(g)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

        def replay(i):
            graphs[i].replay()
            return static_loss[i]

        graph_time, glosses = run_epochs([lambda i=i: replay(i) for i in range(len(batches))])
        result.update({"epoch_time_s": graph_time, "timing": "each training iteration replayed from a CUDA graph",
                       "last_loss": glosses[-1]})
        graphs.clear()
    if reducer is not None:
        reducer.remove_hooks()
    return result


def training_step_ms(rank, world, dev, sequence_parallel, iters=30):
    """Milliseconds of one full training iteration of the node-level Graphormer (4 layers, hidden 64, 8
    heads, 128 features, 40 classes; forward, nll_loss, backward, gradient averaging, fused AdamW) with
    64,000 nodes on every rank, replayed from a CUDA graph and timed with CUDA events, max over ranks.
    ``sequence_parallel=True``: the ranks share one graph of world x 64,000 nodes (Ulysses layer, weights
    replicated, gradients averaged); False: every rank trains its own 64,000-node graph with all heads and
    no communication — the single-GPU iteration measured in the same job on the same GPUs."""
    import torch.distributed as dist
    from torch.nn import functional as F
    from torchgt_b200 import SparseGraph
    from torchgt_b200.graphormer import Graphormer
    from torchgt_b200.gt_sp import initialize as sp
    from torchgt_b200.gt_sp.reducer import Reducer
    from torchgt_b200.gt_sp.utils import adjust_edge_index_nomerge
    from torchgt_b200.synthetic import benchmark_64k
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.manual_seed(42)
    L = NODES_PER_RANK
    shared = sequence_parallel and world > 1
    model = Graphormer(4, 8, 128, 64, 40, 1, 0.3, 0.1, 0.5, 64, 1).to(dev).train()
    if not shared:
        for layer in model.layers:
            layer.self_attention.sequence_parallel = False
    elif world > 1:
        for p in model.parameters():
            dist.broadcast(p.data, src=0)
    opt = torch.optim.AdamW(model.parameters(), lr=2e-4, weight_decay=0.01, fused=True, capturable=True)
    reducer = Reducer().init(model) if shared else None
    ei, n_rows = benchmark_64k(ranks=world if shared else 1)
    if shared:
        ei = adjust_edge_index_nomerge(ei, L)
        n_rows = world * (L + 1)
        sp.set_global_token_indices(list(range(0, n_rows, L + 1)))
    graph = SparseGraph(ei.to(dev), n_rows)
    graph.by_src
    gen = torch.Generator().manual_seed(7 + rank)
    x = torch.randn(L, 128, generator=gen).to(dev)
    y = torch.randint(0, 40, (L,), generator=gen).to(dev)

    def iteration():
        loss = F.nll_loss(model(x, None, graph, attn_type="sparse"), y)
        if reducer is not None:
            reducer.prepare()
            loss.backward()
            reducer.synchronize()
        else:
            opt.zero_grad(set_to_none=True)
            loss.backward()
        opt.step()
        return loss

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            iteration()
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        loss = iteration()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        g.replay()
    stop.record()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(stop) / iters], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    last = float(loss.detach())
    del g
    if reducer is not None:
        reducer.remove_hooks()
    return float(ms.item()), last


def weak_scaling_step(rank, world, dev):
    """The end-to-end training step under weak scaling: 64,000 nodes per rank, the whole model around the
    layer.  Efficiency = single-GPU iteration time / N-GPU iteration time, both measured in this job."""
    single_ms, _ = training_step_ms(rank, world, dev, sequence_parallel=False)
    if world == 1:
        return {"nodes_per_rank": NODES_PER_RANK, "ms_per_iteration": single_ms, "single_gpu_ms_per_iteration": single_ms,
                "efficiency": 1.0, "target_efficiency": 0.85}
    multi_ms, loss = training_step_ms(rank, world, dev, sequence_parallel=True)
    return {"nodes_per_rank": NODES_PER_RANK, "n_gpus": world, "ms_per_iteration": multi_ms,
            "single_gpu_ms_per_iteration": single_ms, "efficiency": single_ms / multi_ms, "target_efficiency": 0.85,
            "sequence_parallel_overhead_ms": multi_ms - single_ms,
            "last_loss": loss,
            "note": "the overhead (exchange over NVLink, barriers, narrower head slices, gradient all-reduce) is a "
                    "fixed number of milliseconds per iteration; the ratio fell when the single-GPU iteration went "
                    "from 8.0 to 2.7 ms with this library's LayerNorm and weight-gradient kernels (both sides of the "
                    "ratio use them), the N-GPU iteration itself got faster",
            "what": "node-level Graphormer (4 layers, hidden 64, 8 heads, 128 features, 40 classes) forward + loss + "
                    "backward + flat gradient all-reduce + fused AdamW per iteration, CUDA-graph replay, CUDA-event "
                    "time, max over ranks; the single-GPU figure is the same iteration on 64,000 nodes with all 8 "
                    "heads and no exchange, run on every GPU of this job at the same time"}


# ---------------------------------------------------------------------------------------------------
class OpBuffers:
    """Device tensors of one input set for direct C-ABI calls (nothing allocated inside the timing)."""

    def __init__(self, graph, dtype, seed, with_bias=True, want_dbias=True, woven_kv=False):
        from torchgt_b200 import _cabi
        dev = graph.device
        n, e = graph.n_rows, graph.n_edges
        self.q, self.k, self.v, self.dout, bias = make_inputs(n, e, dtype, seed, dev)
        self.row_bytes = HEADS * HEAD_DIM * self.q.element_size()
        self.kv_row_bytes = self.row_bytes
        if woven_kv:   # K and V of a row side by side, as the sequence-parallel exchange can deliver them
            self.kv = torch.stack([self.k, self.v], dim=1).contiguous()        # [n, 2, H, D]
            self.k, self.v = self.kv[:, 0], self.kv[:, 1]
            self.kv_row_bytes = 2 * self.row_bytes
        self.bias = bias if with_bias else None
        self.out = torch.empty_like(self.q)
        self.z = torch.empty(n, HEADS, dtype=torch.float32, device=dev)
        self.dq, self.dk, self.dv = (torch.empty_like(self.q) for _ in range(3))
        self.dbias = torch.empty_like(bias) if (with_bias and want_dbias) else None
        lib = _cabi.load()
        nb = ctypes.c_size_t()
        self.code = _cabi.TGT_F32 if dtype == torch.float32 else _cabi.TGT_BF16
        _cabi.check(lib.tgt_sparse_attn_scratch_bytes(graph.by_dst.byref(), graph.by_src.byref(), HEADS, HEAD_DIM,
                                                      self.code, 1, ctypes.byref(nb)))
        nf = ctypes.c_size_t()
        _cabi.check(lib.tgt_sparse_attn_scratch_bytes(graph.by_dst.byref(), None, HEADS, HEAD_DIM, self.code, 0,
                                                      ctypes.byref(nf)))
        self.scratch_f = torch.empty(max(nf.value, 16), dtype=torch.uint8, device=dev)
        self.scratch_b = torch.empty(max(nb.value, 16), dtype=torch.uint8, device=dev)
        self.graph = graph

    def fwd(self, stream):
        from torchgt_b200 import _cabi
        lib = _cabi.load()
        p = lambda t: None if t is None else t.data_ptr()
        _cabi.check(lib.tgt_sparse_attn_fwd_strided(
            p(self.q), self.row_bytes, p(self.k), p(self.v), self.kv_row_bytes, p(self.bias),
            1 if self.bias is not None else 0, self.graph.by_dst.byref(), p(self.out), p(self.z), HEADS, HEAD_DIM,
            self.code, p(self.scratch_f), self.scratch_f.numel(), stream))

    def bwd(self, stream, passes):
        from torchgt_b200 import _cabi
        lib = _cabi.load()
        p = lambda t: None if t is None else t.data_ptr()
        _cabi.check(lib.tgt_sparse_attn_bwd_strided(
            p(self.dout), self.row_bytes, p(self.q), self.row_bytes, p(self.k), p(self.v), self.kv_row_bytes,
            p(self.bias), 1 if self.bias is not None else 0, p(self.out), p(self.z), self.graph.by_dst.byref(),
            self.graph.by_src.byref(), p(self.dq), p(self.dk), p(self.dv), p(self.dbias), HEADS, HEAD_DIM, self.code,
            p(self.scratch_b), self.scratch_b.numel(), stream, passes))


def capture(fn):
    """Capture the launches ``fn(stream)`` makes into a CUDA graph."""
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn(side.cuda_stream)      # warm-up outside capture (module load, first-launch work)
    side.synchronize()
    with torch.cuda.graph(g, stream=side):
        fn(torch.cuda.current_stream().cuda_stream)
    return g


def kernels_per_step(graph, with_dbias=True, ranks=1, elem=4):
    # forward, dQ pass, dK/dV pass: one kernel each, plus a second small kernel each where rows are at most
    # 64 bytes wide (there the rows that cross tiles are finished separately); the row-statistics pre-pass
    # runs only when dbias is computed
    row_bytes = HEADS // max(1, ranks) * HEAD_DIM * elem
    return 3 * (2 if row_bytes <= 64 else 1) + (1 if with_dbias else 0)


def measure_device_resident(sets, steps, warmup):
    """CUDA-event timings of forward+backward through the C ABI on device-resident input sets: the whole
    step (with dbias), the step with the bias as a plain input, and each phase on its own."""
    import copy
    n_sets = len(sets)
    step_graphs = [capture(lambda s, b=b: (b.fwd(s), b.bwd(s, 7 if b.dbias is not None else 6))) for b in sets]
    phase_graphs = [[capture(lambda s, b=b: b.fwd(s)), capture(lambda s, b=b: b.bwd(s, 3 if b.dbias is not None else 2)),
                     capture(lambda s, b=b: b.bwd(s, 4))] for b in sets]
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(graphs):
        for i in range(warmup):
            graphs[i % n_sets].replay()
        torch.cuda.synchronize()
        start.record()
        for i in range(steps):
            graphs[i % n_sets].replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps

    # ---- device-resident throughput: K back-to-back steps over rotating input sets -------------------
    ms_per_step = timed(step_graphs)
    # ---- the same step with the bias as a plain input (no dbias: no statistics pre-pass) ---------------
    plain_sets = []
    for b in sets:
        b2 = copy.copy(b)
        b2.dbias = None
        plain_sets.append(b2)
    plain_graphs = [capture(lambda s, b=b: (b.fwd(s), b.bwd(s, 6))) for b in plain_sets]
    ms_no_dbias = timed(plain_graphs)
    plain_graphs.clear()
    # ---- per-phase durations (each phase its own graph, events around every replay) ------------------
    names = ["fwd_kernel", "bwd_dq_kernel", "bwd_dkv_kernel"]
    phase_steps = min(steps, 200)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(phase_steps)]
    for i in range(phase_steps):
        for j in range(3):
            evs[i][j].record()
            phase_graphs[i % n_sets][j].replay()
        evs[i][3].record()
    torch.cuda.synchronize()
    phase_ms = {n: statistics.mean(evs[i][j].elapsed_time(evs[i][j + 1]) for i in range(phase_steps))
                for j, n in enumerate(names)}
    return {"ms_per_step": ms_per_step, "ms_no_dbias": ms_no_dbias, "phase_ms": phase_ms, "names": names}


def extra_workload(name, dtype, steps, warmup, zipf=None):
    """One more single-GPU workload of the metric, timed like the headline (device-resident, CUDA graph,
    rotating input sets) with fewer steps: returns a small record for the bench line."""
    from torchgt_b200 import SparseGraph
    from torchgt_b200.synthetic import benchmark_64k, benchmark_870k
    dev = torch.device("cuda", 0)
    if name == "870k":
        edge_index, n_rows = benchmark_870k() if zipf is None else benchmark_870k(zipf_exponent=zipf)
    else:
        edge_index, n_rows = benchmark_64k()
    n_edges = edge_index.shape[1]
    graph = SparseGraph(edge_index.to(dev), n_rows)
    graph.by_src
    del edge_index
    n_sets = 3 if name == "870k" else ROTATING_SETS
    sets = [OpBuffers(graph, dtype, 1234 + i) for i in range(n_sets)]
    sampler = ClockSampler(0)
    m = measure_device_resident(sets, steps, warmup)
    clocks = sampler.stop()
    elem = 4 if dtype == torch.float32 else 2
    peak, peak_kind = measured_hbm_peak()
    bytes_ = algorithmic_bytes(n_rows, n_edges, HEADS, HEAD_DIM, elem, 4)
    dominant = max(m["names"], key=lambda n: m["phase_ms"][n])
    step_bytes = sum(bytes_.values())
    del sets, graph
    torch.cuda.empty_cache()
    return {"rows": n_rows, "edges": n_edges, "io_dtype": "fp32" if elem == 4 else "bf16", "steps": steps,
            "ms_per_step": m["ms_per_step"], "edges_per_s": n_edges / (m["ms_per_step"] * 1e-3),
            "frac": step_bytes / (m["ms_per_step"] * 1e-3) / 1e9 / peak, "peak_kind": f"of {peak_kind}",
            "dominant_phase": dominant,
            "dominant_phase_frac": bytes_[dominant] / (m["phase_ms"][dominant] * 1e-3) / 1e9 / peak,
            "phases_ms": m["phase_ms"],
            "phases_frac": {n: bytes_[n] / (m["phase_ms"][n] * 1e-3) / 1e9 / peak for n in m["names"]},
            "ms_per_step_without_dbias": m["ms_no_dbias"], "clocks": clocks}


def run_single_gpu(args, dtype):
    from torchgt_b200 import SparseGraph, sparse_graph_attention
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.profile and args.slice_of > 1:
        # the head slice one rank of an N-rank sequence-parallel run sees: N x 64,000 nodes, 8 / N heads
        global HEADS
        from torchgt_b200.gt_sp.utils import adjust_edge_index_nomerge
        edge_index, _ = load_workload("64k", ranks=args.slice_of)
        edge_index = adjust_edge_index_nomerge(edge_index, NODES_PER_RANK)
        n_rows = args.slice_of * (NODES_PER_RANK + 1)
        HEADS = HEADS // args.slice_of
    else:
        edge_index, n_rows = load_workload(args.workload)
    n_edges = edge_index.shape[1]
    graph = SparseGraph(edge_index.to(dev), n_rows)
    graph.by_src  # build both layouts before timing
    sets = [OpBuffers(graph, dtype, 1234 + i, with_bias=not (args.profile and args.no_bias))
            for i in range(ROTATING_SETS)]
    if args.profile:
        # plain launches of a few steps for ncu (no CUDA graph, no end-to-end or CPU legs)
        stream = torch.cuda.current_stream().cuda_stream
        for i in range(args.warmup + args.steps):
            sets[i % ROTATING_SETS].fwd(stream)
            sets[i % ROTATING_SETS].bwd(stream, 7 if sets[i % ROTATING_SETS].dbias is not None else 6)
        torch.cuda.synchronize()
        print(json.dumps({"profile_run": True, "steps": args.steps, "warmup": args.warmup, "rows": n_rows,
                          "edges": n_edges, "heads": HEADS, "bias": not args.no_bias}), flush=True)
        return
    sampler = ClockSampler(0)
    m = measure_device_resident(sets, args.steps, args.warmup)
    ms_per_step, ms_no_dbias, phase_ms, names = m["ms_per_step"], m["ms_no_dbias"], m["phase_ms"], m["names"]

    # ---- end to end through the public API from pinned host memory -----------------------------------
    hq, hk, hv, hdout, hbias = (t.pin_memory() for t in make_inputs(n_rows, n_edges, dtype, 99, None))
    hei = edge_index.to(torch.int32).pin_memory()   # the layouts are built from int32 ids: 8 bytes per edge on the bus
    host_out = [torch.empty_like(hq).pin_memory() for _ in range(4)]
    host_dbias = torch.empty_like(hbias).pin_memory()

    def e2e_step(resident_graph=None):
        q, k, v = (t.to(dev, non_blocking=True).requires_grad_() for t in (hq, hk, hv))
        bias = hbias.to(dev, non_blocking=True).requires_grad_()
        dout = hdout.to(dev, non_blocking=True)
        g = resident_graph if resident_graph is not None else SparseGraph(hei.to(dev, non_blocking=True), n_rows)
        out = sparse_graph_attention(q, k, v, g, bias)
        out.backward(dout)
        for dst, src in zip(host_out, (out.detach(), q.grad, k.grad, v.grad)):
            dst.copy_(src, non_blocking=True)
        host_dbias.copy_(bias.grad, non_blocking=True)
        torch.cuda.synchronize()

    e2e_steps = max(3, min(args.steps, 30))
    results = {}
    for label, g in (("full", None), ("graph_resident", graph)):
        for _ in range(3):
            e2e_step(g)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step(g)
        results[label] = (time.perf_counter() - t0) / e2e_steps

    # The same per-step work issued on a few streams in rotation (each with its own pinned result
    # buffers), so that the upload of one step overlaps the download of the previous one: PCIe is full
    # duplex and the step is transfer-bound.  Every step still uploads all its inputs and downloads all
    # its results.
    n_streams = int(os.environ.get("TGT_BENCH_E2E_STREAMS", "4"))
    streams = [torch.cuda.Stream() for _ in range(n_streams)]
    host_out2 = [[torch.empty_like(hq).pin_memory() for _ in range(4)] for _ in streams]
    host_dbias2 = [torch.empty_like(hbias).pin_memory() for _ in streams]

    def e2e_step_async(i):
        st = streams[i % n_streams]
        with torch.cuda.stream(st):
            q, k, v = (t.to(dev, non_blocking=True).requires_grad_() for t in (hq, hk, hv))
            bias = hbias.to(dev, non_blocking=True).requires_grad_()
            dout = hdout.to(dev, non_blocking=True)
            g = SparseGraph(hei.to(dev, non_blocking=True), n_rows)   # builds without a host synchronisation
            out = sparse_graph_attention(q, k, v, g, bias)
            out.backward(dout)
            for dst, src in zip(host_out2[i % n_streams], (out.detach(), q.grad, k.grad, v.grad)):
                dst.copy_(src, non_blocking=True)
            host_dbias2[i % n_streams].copy_(bias.grad, non_blocking=True)

    for i in range(4):
        e2e_step_async(i)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step_async(i)
    torch.cuda.synchronize()
    results["pipelined"] = (time.perf_counter() - t0) / e2e_steps
    clocks = sampler.stop()

    elem = 4 if dtype == torch.float32 else 2
    h2d = 4 * n_rows * HEADS * HEAD_DIM * elem + n_edges * 4 + 2 * n_edges * 4
    d2h = 4 * n_rows * HEADS * HEAD_DIM * elem + n_edges * 4
    peak, peak_kind = measured_hbm_peak()
    bytes_ = algorithmic_bytes(n_rows, n_edges, HEADS, HEAD_DIM, elem, 4)
    dominant = max(names, key=lambda n: phase_ms[n])
    achieved = bytes_[dominant] / (phase_ms[dominant] * 1e-3) / 1e9
    step_bytes = sum(bytes_.values())
    step_achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    cpu, _ = cpu_reference_rate(edge_index, n_rows, steps=5, warmup=2, time_limit_s=20.0)
    epoch = None
    if dtype == torch.float32 and os.environ.get("TGT_BENCH_EPOCH", "1") != "0":
        try:
            epoch = epoch_benchmark(0, 1, dev, args.workload)
        except Exception as exc:          # the headline numbers above do not depend on this leg
            epoch = {"error": repr(exc)[:300]}
    # the rest of the metric (870K sequence length, bf16), timed the same way with fewer steps
    more = None
    if args.workload == "64k" and dtype == torch.float32 and os.environ.get("TGT_BENCH_MORE", "1") != "0":
        del sets
        torch.cuda.empty_cache()
        more = {}
        for key, wl, dt, zipf in (("64k_bf16", "64k", torch.bfloat16, None), ("870k_fp32", "870k", torch.float32, None),
                                  ("870k_fp32_uniform_sources", "870k", torch.float32, 0.0),
                                  ("870k_bf16", "870k", torch.bfloat16, None)):
            try:
                more[key] = extra_workload(wl, dt, 40 if wl == "870k" else 200, 5, zipf)
            except Exception as exc:
                more[key] = {"error": repr(exc)[:300]}
        more["note"] = ("same timing as the headline (device-resident forward+backward with dbias through the C ABI, "
                        "CUDA graph, rotating input sets larger than L2); 870k = 870,001 rows, 18,214,272 edges; "
                        "uniform_sources draws the random edges' sources uniformly instead of from the power law, "
                        "so no K/V row is hot in L2")
    line = {
        "metric": "sparse_graph_attention_fwd_bwd_edges_per_s", "value": n_edges / (ms_per_step * 1e-3),
        "unit": "edges/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if dtype == torch.float32 else "bf16 i/o, f32 math", "data": "synthetic",
        "config": workload_config(1, n_rows, n_edges, args.dtype, args.workload),
        "clocks": clocks,
        "e2e": {"value": n_edges / results["pipelined"], "unit": "edges/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": results["pipelined"] * 1e3,
                "includes": "pinned-host uploads of q,k,v,bias,dO and the int32 edge list, both edge layouts "
                            "built, forward, backward, downloads of out,dq,dk,dv,dbias, every step; steps "
                            "rotate over four streams so uploads overlap the previous steps' downloads",
                "one_step_at_a_time_value": n_edges / results["full"],
                "one_step_at_a_time_ms": results["full"] * 1e3,
                "graph_resident_value": n_edges / results["graph_resident"],
                "graph_resident_ms_per_step": results["graph_resident"] * 1e3},
        "gpu_launches": kernels_per_step(graph, elem=elem) * args.steps,
        "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                     "traffic": (ncu_traffic(args.workload, args.dtype) or {}).get(dominant),
                     "algorithmic_bytes_per_launch": bytes_[dominant],
                     "phases_ms": phase_ms,
                     "phases_frac": {n: bytes_[n] / (phase_ms[n] * 1e-3) / 1e9 / peak for n in names},
                     "step": {"algorithmic_bytes": step_bytes, "achieved": step_achieved,
                              "frac": step_achieved / peak, "frac_of_nominal_8TBs": step_achieved / 8000.0},
                     "step_without_dbias": {
                         "ms_per_step": ms_no_dbias, "edges_per_s": n_edges / (ms_no_dbias * 1e-3),
                         "frac": step_bytes / (ms_no_dbias * 1e-3) / 1e9 / peak,
                         "note": "bias read as an input, its gradient not computed (the byte count has no dbias "
                                 "term either); the headline step computes dbias as well"}},
        "cpu_baseline": cpu,
        "epoch": epoch,
        "more_workloads": more,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
def rank_inputs(rank, i, L, dtype):
    """The seeded q, k, v [1, L+1, H, D] and dO [1, L+1, H*D] of rank ``rank``, input set ``i`` (host)."""
    gen = torch.Generator().manual_seed(4321 + 17 * rank + i)
    q, k, v = (torch.randn(1, L + 1, HEADS, HEAD_DIM, generator=gen).to(dtype) for _ in range(3))
    dout = torch.randn(1, L + 1, HEADS * HEAD_DIM, generator=gen).to(dtype)
    return q, k, v, dout


def layer_parity(layer, graph, edge_index, rank, world, L, dev, dtype):
    """One forward+backward of the layer on every rank, compared with the float64 CPU oracle (outside any
    timed region).  Every output row depends only on its in-edges and every dK/dV row on its out-edges and
    on the statistics of their destinations, so a sample of rows is checked EXACTLY against the oracle
    evaluated on the sub-problem that holds all those edges; the global-token row 0 (in- and out-degree
    world x 64,000) is always in the sample.  Each rank checks its own rows for two of the eight heads
    (rank r: heads r mod 8 and (r + 3) mod 8, so every rank's attention kernels are covered).
    Returns the largest error relative to max |reference| of each compared tensor."""
    import numpy as np
    import torch.distributed as dist
    from oracle.sparse_attn_oracle import backward_closed_form, forward_closed_form
    heads = sorted({rank % HEADS, (rank + 3) % HEADS})
    full = [rank_inputs(r, 0, L, dtype) for r in range(world)]
    cat = lambda j: torch.cat([f[j][0].float() for f in full], dim=0)
    q_all, k_all, v_all = (cat(j)[:, heads].contiguous() for j in range(3))                # [N, 2, D]
    do_all = cat(3).view(-1, HEADS, HEAD_DIM)[:, heads].contiguous()
    slots = [r * (L + 1) for r in range(world)]
    # copy_global_token0: every rank's slot of the global token reads row 0's output, so row 0 collects
    # their gradients and the slots' own rows get none
    do_eff = do_all.clone()
    do_eff[0] = do_all[slots].sum(dim=0)
    do_eff[slots[1:]] = 0

    q, k, v, dout = (t.to(dev) for t in full[rank])
    q, k, v = (t.requires_grad_() for t in (q, k, v))
    out = layer(q, k, v, None, graph, "sparse")
    out.backward(dout)
    torch.cuda.synchronize()
    mine = {"out": out.detach(), "dq": q.grad, "dk": k.grad, "dv": v.grad}
    mine = {n: t.float().cpu().view(L + 1, HEADS, HEAD_DIM)[:, heads].double().numpy() for n, t in mine.items()}

    gen = torch.Generator().manual_seed(99 + rank)
    base = rank * (L + 1)
    local_dst = torch.randint(1, L + 1, (192,), generator=gen).unique()
    local_src = torch.randint(1, L + 1, (64,), generator=gen).unique()
    n_total = world * (L + 1)
    is_src = torch.zeros(n_total, dtype=torch.bool); is_src[base + local_src] = True
    dests = edge_index[1][is_src[edge_index[0]]].unique()
    is_dst = torch.zeros(n_total, dtype=torch.bool)
    is_dst[base + local_dst] = True; is_dst[dests] = True; is_dst[0] = True
    sub = edge_index[:, is_dst[edge_index[1]]]
    ref_out, _ = forward_closed_form(q_all, k_all, v_all, sub)
    ref_dq, ref_dk, ref_dv, _ = backward_closed_form(q_all, k_all, v_all, sub, do_eff)

    def err(x, ref):
        return float(np.abs(x - ref).max() / max(np.abs(ref).max(), 1e-30))

    errs = {}
    d_rows = local_dst.numpy()
    errs["out"] = max(err(mine["out"][d_rows], ref_out[base + d_rows]),
                      err(mine["out"][0], ref_out[0]))               # this rank's token slot = row 0's output
    errs["dq"] = err(mine["dq"][d_rows], ref_dq[base + d_rows])
    if rank == 0:
        errs["dq"] = max(errs["dq"], err(mine["dq"][0], ref_dq[0]))
    else:
        errs["dq"] = max(errs["dq"], float(np.abs(mine["dq"][0]).max()))   # the other slots have no edges
    s_rows = local_src.numpy()
    errs["dk"] = err(mine["dk"][s_rows], ref_dk[base + s_rows])
    errs["dv"] = err(mine["dv"][s_rows], ref_dv[base + s_rows])
    if rank == 0:   # row 0's out-edges reach every node: their destinations are not all in the sample; its
        pass        # in-edge side (out, dq) is checked above
    worst = torch.tensor([errs["out"], errs["dq"], errs["dk"], errs["dv"]], device=dev, dtype=torch.float64)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    worst = worst.tolist()
    return {"max_rel_err": max(worst), "out": worst[0], "dq": worst[1], "dk": worst[2], "dv": worst[3],
            "rows": int(local_dst.numel() + 1), "source_rows": int(local_src.numel()), "edges_in_subproblem": int(sub.shape[1]),
            "heads_checked_per_rank": 2, "tolerance": 1e-5 if dtype == torch.float32 else 1e-2,
            "oracle": "float64 closed form of the reference's op sequence (oracle/sparse_attn_oracle.py)"}


def run_multi_gpu(args, dtype, rank, world):
    import gc
    import torch.distributed as dist
    from torchgt_b200 import CoreAttention, SparseGraph
    from torchgt_b200.gt_sp import initialize as sp
    from torchgt_b200.gt_sp import p2p
    from torchgt_b200.gt_sp.layer import DistributedAttentionNoMerge
    from torchgt_b200.gt_sp.utils import adjust_edge_index_nomerge
    from torchgt_b200.synthetic import benchmark_64k
    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    sp.set_global_token_num(1)
    sp.initialize_sequence_parallel(NODES_PER_RANK * world, 1, 1, world)
    L = NODES_PER_RANK
    sp.set_global_token_indices(list(range(0, world * (L + 1), L + 1)))
    edge_index, _ = benchmark_64k(ranks=world)                       # ids 0..S, same on every rank
    edge_index = adjust_edge_index_nomerge(edge_index, L)
    n_rows, n_edges = world * (L + 1), edge_index.shape[1]
    graph = SparseGraph(edge_index.to(dev), n_rows)
    graph.by_src
    core = CoreAttention(HEADS * HEAD_DIM, 0.0, HEADS, 1)
    layer = DistributedAttentionNoMerge(core, sp.get_sequence_parallel_group()).train()

    def note(msg):
        if os.environ.get("TGT_BENCH_TRACE"):
            print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)

    # ---- parity first: the numbers below are only worth something if the layer is right -----------------
    parity = layer_parity(layer, graph, edge_index, rank, world, L, dev, dtype)
    px = p2p.peer_exchange_for(sp.get_sequence_parallel_group(), dev)
    parity["transport"] = "p2p" if px is not None else "nccl"
    note(f"parity {parity['max_rel_err']:.2e}")
    if parity["max_rel_err"] > parity["tolerance"]:
        if rank == 0:
            print(json.dumps({"error": "multi-GPU parity failed", "parity": parity}), flush=True)
        dist.barrier()
        p2p.reset_peer_exchanges()
        dist.destroy_process_group()
        raise SystemExit(3)

    sets = []
    for i in range(ROTATING_SETS):
        q, k, v, dout = (t.to(dev) for t in rank_inputs(rank, i, L, dtype))
        sets.append((q.requires_grad_(), k.requires_grad_(), v.requires_grad_(), dout))

    def step(i):
        q, k, v, dout = sets[i % ROTATING_SETS]
        out = layer(q, k, v, None, graph, "sparse")
        out.backward(dout)
        q.grad = k.grad = v.grad = None

    def timed(fn):
        for i in range(args.warmup):
            fn(i)
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(args.steps):
            fn(i)
        stop.record()
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        ms = torch.tensor([start.elapsed_time(stop) / args.steps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local) if rank == 0 else None
    eager_ms = timed(step)
    note(f"eager {eager_ms:.3f} ms")
    # The same step (layer forward, backward, both exchanges) captured once per input set in a CUDA
    # graph: every kernel of the exchange and of the attention replays without host work in between.
    graphs = []
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(ROTATING_SETS):
            step(i)
    side.synchronize(); dist.barrier()
    for i in range(ROTATING_SETS):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            step(i)
        graphs.append(g)
    torch.cuda.synchronize(); dist.barrier()
    ms_per_step = timed(lambda i: graphs[i % ROTATING_SETS].replay())
    p2p.check_peer_exchanges()           # a barrier that gave up on a peer invalidates the timing
    note(f"graph {ms_per_step:.3f} ms")

    # TGT_BENCH_KERNEL_LIST=1: device time of every kernel of the replayed step on rank 0, from the CUPTI
    # activity records torch.profiler collects (a per-rank tool: every rank runs the same replays).  The
    # kernels of a chain of dependent launches start before their predecessor ends, so their times overlap.
    kernel_list = None
    if os.environ.get("TGT_BENCH_KERNEL_LIST"):
        from torch.profiler import ProfilerActivity, profile
        reps = 2 * ROTATING_SETS
        torch.cuda.synchronize(); dist.barrier()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(reps):
                graphs[i % ROTATING_SETS].replay()
            torch.cuda.synchronize()
        # median duration per kernel name (the first replays wait at their barriers for the rank whose
        # profiler started last, which a mean would charge to the barrier kernel)
        from torch.autograd import DeviceType
        per_name = {}
        for e in prof.events():
            if e.device_type == DeviceType.CUDA and e.device_time_total > 0:
                per_name.setdefault(e.name, []).append(e.device_time_total)
        kernel_list = sorted(({"kernel": name[:100], "launches_per_step": len(d) / reps,
                               "us_per_step": statistics.median(d) * len(d) / reps} for name, d in per_name.items()),
                             key=lambda r: -r["us_per_step"])
        dist.barrier()

    # the exchange alone: the data movement of one step (both pushes, four barriers, both pulls) with the
    # attention kernels left out, captured and replayed like the step itself
    exchange_ms = None
    if px is not None:
        heads_l = HEADS // world
        row_bytes = heads_l * HEAD_DIM * sets[0][0].element_size()
        tensor_bytes = n_rows * row_bytes
        rows_dev = sp.get_global_token_rows_on(dev)
        scratch_out = torch.empty(1, L + 1, HEADS * HEAD_DIM, dtype=dtype, device=dev)
        scratch_grads = [torch.empty(1, L + 1, HEADS, HEAD_DIM, dtype=dtype, device=dev) for _ in range(3)]

        def exchange_step(i):
            q, k, v, dout = sets[i % ROTATING_SETS]
            qkv = px.acquire(3 * tensor_bytes)
            px.push([q.detach(), k.detach(), v.detach()], qkv, L + 1, row_bytes, (L + 1) * row_bytes)
            px.barrier()
            landing = px.acquire(tensor_bytes, p2p.SOURCE)
            px.barrier()
            px.pull(landing, [scratch_out], 1, L + 1, row_bytes, rows_dev)
            px.release(landing)
            landing = px.acquire(tensor_bytes)
            px.push([dout], landing, L + 1, row_bytes, (L + 1) * row_bytes)
            px.barrier()
            grads = px.acquire(3 * tensor_bytes, p2p.SOURCE)
            px.release(qkv); px.release(landing)
            px.barrier()
            px.pull(grads, scratch_grads, 1, L + 1, row_bytes)
            px.release(grads)

        with torch.cuda.stream(side):
            for i in range(ROTATING_SETS):
                exchange_step(i)
        side.synchronize(); dist.barrier()
        ex_graphs = []
        for i in range(ROTATING_SETS):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                exchange_step(i)
            ex_graphs.append(g)
        torch.cuda.synchronize(); dist.barrier()
        exchange_ms = timed(lambda i: ex_graphs[i % ROTATING_SETS].replay())
        ex_graphs.clear()
        p2p.check_peer_exchanges()

    # the attention alone (no exchange) on this rank's head slice of the same graph, for reference
    heads_local = HEADS // world
    op_sets = []
    for i in range(ROTATING_SETS):
        gen = torch.Generator().manual_seed(99 + i)
        t = [torch.randn(n_rows, heads_local, HEAD_DIM, generator=gen).to(dtype).to(dev).requires_grad_()
             for _ in range(3)]
        op_sets.append((t, torch.randn(n_rows, heads_local, HEAD_DIM, generator=gen).to(dtype).to(dev)))

    def op_step(i):
        (q, k, v), dout = op_sets[i % ROTATING_SETS]
        from torchgt_b200 import sparse_graph_attention
        sparse_graph_attention(q, k, v, graph).backward(dout)
        q.grad = k.grad = v.grad = None

    with torch.cuda.stream(side):
        for i in range(ROTATING_SETS):
            op_step(i)
    side.synchronize()
    op_graphs = []
    for i in range(ROTATING_SETS):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            op_step(i)
        op_graphs.append(g)
    torch.cuda.synchronize(); dist.barrier()
    op_ms = timed(lambda i: op_graphs[i % ROTATING_SETS].replay())
    del op_sets

    # end to end: this rank's q, k, v, dO come from pinned host memory, the result goes back
    host = [t.detach().cpu().pin_memory() for t in sets[0]]
    host_out = [torch.empty_like(host[0].view(1, L + 1, -1)).pin_memory()] + \
               [torch.empty_like(host[0]).pin_memory() for _ in range(3)]

    def e2e_step():
        q, k, v = (t.to(dev, non_blocking=True).requires_grad_() for t in host[:3])
        dout = host[3].to(dev, non_blocking=True)
        out = layer(q, k, v, None, graph, "sparse")
        out.backward(dout)
        for dst, src in zip(host_out, (out.detach(), q.grad, k.grad, v.grad)):
            dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()

    e2e_steps = max(3, min(args.steps, 30))
    for _ in range(3):
        e2e_step()
    dist.barrier(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    dist.barrier()
    e2e_s = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device=dev)
    dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if sampler else None
    epoch = weak = None
    if dtype == torch.float32 and os.environ.get("TGT_BENCH_EPOCH", "1") != "0":
        try:
            epoch = epoch_benchmark(rank, world, dev)
        except Exception as exc:
            epoch = {"error": repr(exc)[:300]}
        try:
            weak = weak_scaling_step(rank, world, dev)
        except Exception as exc:
            weak = {"error": repr(exc)[:300]}
        sp.set_global_token_indices(list(range(0, world * (L + 1), L + 1)))

    if rank == 0:
        elem = 4 if dtype == torch.float32 else 2
        peak, peak_kind = measured_hbm_peak()
        bytes_ = algorithmic_bytes(n_rows, n_edges, heads_local, HEAD_DIM, elem, 0)
        step_bytes = sum(bytes_.values())
        per_rank_io = 4 * (L + 1) * HEADS * HEAD_DIM * elem
        # kernels: the attention phases; per step two pushes, two pulls, four barriers, one global-row kernel
        launches = kernels_per_step(graph, with_dbias=False, ranks=world, elem=elem) + (9 if px is not None else 12)
        line = {
            "metric": "sparse_graph_attention_fwd_bwd_edges_per_s", "value": n_edges / (ms_per_step * 1e-3),
            "unit": "edges/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32" if dtype == torch.float32 else "bf16 i/o, f32 math", "data": "synthetic",
            "config": workload_config(world, n_rows, n_edges, args.dtype),
            "step": {"timing": "step captured in a CUDA graph per input set, replayed",
                     "what": "DistributedAttentionNoMerge fwd+bwd: exchange(q,k,v) -> attention with "
                             f"{heads_local} head(s) over all rows -> exchange(out), reversed in backward",
                     "bias": "none (the models pass attn_bias=None on this path)"},
            "parity": parity,
            "clocks": clocks,
            "e2e": {"value": n_edges / float(e2e_s.item()), "unit": "edges/s", "h2d_bytes_per_step": per_rank_io,
                    "d2h_bytes_per_step": per_rank_io, "ms_per_step": float(e2e_s.item()) * 1e3,
                    "includes": "per rank: pinned-host uploads of q,k,v,dO, layer forward+backward with both "
                                "exchanges, downloads of out,dq,dk,dv; edge layouts resident"},
            "gpu_launches": launches * args.steps,
            "eager_ms_per_step": eager_ms,
            "exchange_only": None if exchange_ms is None else {
                "ms_per_step": exchange_ms,
                "bytes_over_nvlink_per_rank_each_way": int(8 * (L + 1) * HEADS * HEAD_DIM * elem * (world - 1) / world),
                "note": "both pushes, four barriers and both pulls of one step without the attention kernels "
                        "(CUDA graph); the pulls read slots nobody wrote in this leg, the bytes moved are the step's"},
            "epoch": epoch,
            "weak_scaling_training_step": weak,
            "kernel_list": kernel_list,
            "attention_only": {"ms_per_step": op_ms, "value": n_edges / (op_ms * 1e-3), "unit": "edges/s",
                               "note": "same graph, this rank's head slice, no exchange (CUDA graph)",
                               "frac_of_hbm_peak": step_bytes / (op_ms * 1e-3) / 1e9 / peak},
            "roofline": {"bound": "hbm", "kernel": "whole step per GPU (attention phases + exchange)",
                         "achieved": step_bytes / (ms_per_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak, "peak_kind": f"of {peak_kind}",
                         "traffic": None, "algorithmic_bytes_per_launch": step_bytes},
        }
        print(json.dumps(line), flush=True)
    # Orderly exit.  Communicator teardown waits for every CUDA graph that captured one of its collectives,
    # so all graphs go first; then the symmetric-memory slots, then the process group.
    graphs.clear(); op_graphs.clear()
    del layer, sets
    gc.collect()
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    p2p.reset_peer_exchanges()
    gc.collect()
    sys.stdout.flush(); sys.stderr.flush()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--dtype", choices=["fp32", "bf16"], default="fp32")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="64k",
                    help="N=1 only: 64k (default, the headline) or 870k (long-sequence batch)")
    ap.add_argument("--profile", action="store_true",
                    help="N=1 only: launch warmup+steps plain forward+backward steps and exit (for ncu)")
    ap.add_argument("--slice-of", type=int, default=1, choices=[1, 2, 4, 8],
                    help="with --profile: run the head slice one rank of an N-rank run sees (N x 64,000 nodes, 8/N heads)")
    ap.add_argument("--no-bias", action="store_true", help="with --profile: no edge bias (the layer's own call form)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    dtype = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (torchgt_b200 has no CPU path); "
                         "use --impl reference for the CPU baseline")
    if world > 1:
        if world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
        run_multi_gpu(args, dtype, rank, world)
    else:
        if args.gpus != 1:
            raise SystemExit("for --gpus N > 1 launch with torch.distributed.run (one process per GPU)")
        run_single_gpu(args, dtype)


if __name__ == "__main__":
    main()
