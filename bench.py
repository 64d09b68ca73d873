#!/usr/bin/env python
"""Benchmark of the trie-walk attention hot path on B200.

Workload (N GPUs, strong scaling): the depth-32 radix trie of a seeded 1.1M-char order-3 Markov corpus
over 65 symbols (Zipf(1.1) marginals) -- 28.3M char positions -- with 4 heads x 32 (d_model 128), fp32.
One step = one pass of the hot path over every position of the trie for one layer: trie-scoped attention
forward, backward with the deterministic dK/dV reduction, and the mass-weighted per-query loss, unit by
unit (root-child subtrees at N=1, bigram subtrees balanced over ranks at N>1), followed at N>1 by one
NCCL all-reduce of a gradient-sized buffer.  `value` is trie nodes (char positions) per second with
inputs resident in HBM; `e2e` is the same through the host-buffer C-ABI call (every rank at once at N>1); `epoch` is
one whole trainer epoch on the same trie.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2|c1|micro|c4|c5] [--kv f32|bf16]
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: corpus chars, vocab, markov order, trie depth, heads, head_dim, model layers (for the grad buffer)
    "c2": dict(chars=1_100_000, vocab=65, order=3, depth=32, heads=4, head_dim=32, layers=4,
               label="depth-32 radix trie, 1.1M-char order-3 Markov corpus (vocab 65), d_model 128, 4 heads x 32, fp32"),
    "c1": dict(chars=20_000, vocab=65, order=2, depth=8, heads=4, head_dim=16, layers=2,
               label="depth-8 radix trie, 20k-char order-2 Markov corpus (vocab 65), d_model 64, 4 heads x 16, fp32"),
    # the 5M-char configuration: 126M positions; its inputs do not fit one GPU at once, so every launch group reads the
    # same resident input buffers (sized for the largest group)
    "c4": dict(chars=5_000_000, vocab=96, order=3, depth=32, heads=8, head_dim=32, layers=6,
               label="depth-32 radix trie, 5M-char order-3 Markov corpus (vocab 96), d_model 256, 8 heads x 32, fp32"),
    # the deep configuration: 20M chars, depth 128, nodes of count < 2 pruned from depth 4 (run it with --kv bf16)
    # (a plain order-4 Markov source has no long verbatim repeats, so its count>=2 trie ends near depth 24; the corpus
    # therefore carries injected repeats, probability 2^-12 per position, spans of 64..256 symbols; c5_plain is the
    # same source without them, kept for the comparison of the two tries' sizes)
    "c5": dict(chars=20_000_000, vocab=96, order=4, depth=128, heads=6, head_dim=64, layers=8, prune=(2, 4), repeat_log2=12,
               label="depth-128 radix trie pruned at count<2, 20M-char order-4 Markov corpus with injected repeats (vocab 96), d_model 384, 6 heads x 64"),
    "c5_plain": dict(chars=20_000_000, vocab=96, order=4, depth=128, heads=6, head_dim=64, layers=8, prune=(2, 4),
                     label="depth-128 radix trie pruned at count<2, 20M-char order-4 Markov corpus without repeats (vocab 96), d_model 384, 6 heads x 64"),
    # reduced copies of the two above for profiler captures (inputs still larger than L2, a few GB on the device)
    "c2s": dict(chars=50_000, vocab=65, order=3, depth=32, heads=4, head_dim=32, layers=4,
                label="depth-32 radix trie, 50k-char order-3 Markov corpus (vocab 65), d_model 128, 4 heads x 32, fp32"),
    "micro_s": dict(nodes=600_000, depth=64, heads=8, head_dim=64, vocab=65, layers=1,
                    label="attention microbench, reduced: 600k-node tree, depth 64, 8 heads x 64, fp32"),
    "micro": dict(nodes=4_000_000, depth=64, heads=8, head_dim=64, vocab=65, layers=1,
                  label="attention microbench: 4M-node tree, depth 64, geometric(0.35) children, 8 heads x 64, fp32"),
}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def touch_once_bytes(n, D, H, kv_bytes):
    """Bytes that must cross HBM when every row is moved exactly once (per layer): forward reads Q, K, V and writes O
    and lse; backward reads Q, K, V, O, dO, lse and writes dQ, dK, dV (plus one lse-sized vector of slack for the
    row-wise dO.O, which this implementation recomputes instead of storing)."""
    fwd = n * (D * 4 + 2 * D * kv_bytes + D * 4 + H * 4)
    bwd = n * (6 * D * 4 + 2 * D * kv_bytes + 2 * H * 4)
    return fwd, bwd


# DRAM bytes per position (dram__bytes_read.sum + dram__bytes_write.sum of one launch / positions of the launch) of
# the forward kernel and of the backward kernel + reduction, from ncu captures of the reduced workloads (c2s for
# d_model 128, micro_s for d_model 512; traffic grows in proportion to the positions).  Key: (d_model, kv store).
# The captures are summarised in profiles/attn_tile_kernels_c2s_ncu_full.md (d_model 128, float32 store; the dK/dV
# reduction adds 0.70 KB per position) and profiles/attn_kernels_micro_s_ncu_full.md (d_model 512, float32 store).
DRAM_BYTES_PER_POSITION = {
    (128, "f32"): (2.18e3, 4.44e3),
    (512, "f32"): (8.71e3, 17.5e3),
}


def workload_config(args, cfg, total_nodes, world, max_depth=None, depth_hist=None):
    """The `config` object of the JSON line: the same keys and values in the GPU arm and in the reference arm."""
    return {"workload": cfg["label"], "kv_store": args.kv, "positions": total_nodes, "tile": args.tile,
            "partition": "root-child subtrees" if unit_level(args.workload, world) == 1 else f"bigram subtrees, LPT over {world} rank(s)",
            "l2": "inputs (GBs per tensor) far larger than the 126 MB L2",
            "max_depth": max_depth, "positions_per_depth": depth_hist}


def bind_to_gpu_numa_node(index):
    """Bind this process to the CPUs of the NUMA node the GPU hangs off, so that pinned host buffers allocated (and
    first touched) afterwards sit in that node's memory.  Returns a short description for the JSON line."""
    try:
        import torch
        pr = torch.cuda.get_device_properties(index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        def cpu_set(text):
            out = set()
            for part in text.strip().split(","):
                a, _, b = part.partition("-")
                out.update(range(int(a), int(b or a) + 1))
            return out

        if node < 0:
            # sysfs has no node for the device (usual inside a container): ask the driver's topology table for the
            # GPU's CPU affinity instead (read-only query)
            topo = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout.splitlines()
            head = next(ln for ln in topo if "CPU Affinity" in ln)
            cols = [c.strip() for c in head.split("\t")]
            row = next(ln for ln in topo if ln.startswith(f"GPU{index}\t") or ln.startswith(f"GPU{index} "))
            cells = [c.strip() for c in row.split("\t")]
            cpus = cpu_set(cells[cols.index("CPU Affinity")])
            node = cells[cols.index("NUMA Affinity")] if "NUMA Affinity" in cols else None
        else:
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                cpus = cpu_set(f.read())
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return {"node": node, "bound": False, "why": "none of the node's CPUs is in this process's affinity mask"}
        os.sched_setaffinity(0, allowed)
        return {"node": node, "bound": True, "cpus": len(allowed)}
    except Exception as e:  # sysfs not visible in the container, or no such attribute
        return {"node": None, "bound": False, "why": f"{type(e).__name__}: {e}"[:120]}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------------------
# workload construction (host)
# ----------------------------------------------------------------------------------------------------------
class Unit:
    """One root-child or bigram subtree: its local tree plus the loss index arrays of its radix nodes."""
    __slots__ = ("parent", "n", "tokens", "q2n", "qoff", "radix_ids", "mass_w", "n_ctx")


def unit_level(wl, world):
    """Root-child units on one rank, bigram units on several -- and always for the 126M-position and the deep configurations, whose
    largest root child (a quarter of all positions) would not fit one GPU as a single launch."""
    return 2 if (world > 1 or wl in ("c4", "c5", "c5_plain")) else 1


def build_units(wl, rank, world, log, single_unit=False, group_rows=4_000_000, device=None):
    import agpt_b200 as A
    cfg = WORKLOADS[wl]
    t0 = time.time()
    if wl.startswith("micro"):
        parent = A.synth_tree(cfg["nodes"], cfg["depth"], 65, 0.35, 65, 75_000, 0)
        token = (np.arange(parent.size) % cfg["vocab"]).astype(np.int32)
        radix_of = np.arange(1, parent.size + 1, dtype=np.int32)          # every node its own one-char edge
        edge_mass = np.ones(parent.size + 1, np.int32)
        counts = (np.arange(parent.size + 2, dtype=np.int32), (np.arange(parent.size + 1) % cfg["vocab"]).astype(np.int32),
                  np.ones(parent.size + 1, np.int32))
    else:
        corpus = A.synth_markov_corpus(cfg["chars"], cfg["vocab"], cfg["order"], 0, cfg.get("repeat_log2", 0))
        # the GPU arm orders the suffixes on its device; the CPU arm uses the level-by-level host builder (same arrays)
        level_key = unit_level(wl, world)
        pm, pd = cfg.get("prune", (1, 4))
        trie = (A.RadixTrie.build(corpus, cfg["depth"], level_key, pm, pd) if device is None else
                A.RadixTrie.build_gpu(corpus, cfg["depth"], level_key, pm, pd, device=device))
        parent, token, cdepth, radix_of = trie.char_tree()
        edge_mass = trie.edge_mass
        if cfg.get("repeat_log2") and device is not None:
            # the two tries side by side: with the injected repeats (used) and of the plain source (sizes only)
            plain = A.RadixTrie.build_gpu(A.synth_markov_corpus(cfg["chars"], cfg["vocab"], cfg["order"], 0), cfg["depth"],
                                          level_key, pm, pd, device=device)
            pdep = plain.char_tree()[2]
            deep = lambda d: f"{int((d > 24).sum())} deeper than 24, {int((d > 64).sum())} deeper than 64"  # noqa: E731
            log(f"trie of the corpus with injected repeats: {parent.size} positions ({deep(cdepth)}), {trie.radix_count} radix nodes, "
                f"max depth {int(cdepth.max())}; of the plain corpus: {pdep.size} positions ({deep(pdep)}), {plain.radix_count} radix nodes, "
                f"max depth {int(pdep.max())}")
            del plain, pdep
        counts = (trie.cnt_off.astype(np.int32), trie.cnt_tok, trie.cnt_val)
    log(f"trie built: {parent.size} positions in {time.time() - t0:.1f}s")
    plan = A.WalkerPlan(parent, 64, -1)
    level = unit_level(wl, world)
    ub, ue = plan.units(level)
    if single_unit:       # the whole forest as one launch (profiling); its depth-1 nodes stay roots
        ub, ue = np.array([0], np.int64), np.array([plan.n], np.int64)
    owner = A.partition_lpt(ue - ub, world)
    # Each rank's units are packed, in depth-first order, into launch groups of at most `group_rows` rows: a
    # group is one forest = one walker plan = one launch per kernel, and one loss chunk.
    d2n = plan.dfs_to_node
    pieces, rows = [], 0      # (local parent, global ids, unit start flag) of the group being filled
    units = []

    def flush():
        nonlocal pieces, rows
        if not pieces:
            return
        u = Unit()
        off, pars, idl, ustart = 0, [], [], []
        for pp, ids in pieces:
            pars.append(np.where(pp < 0, -1, pp + off))
            idl.append(ids)
            st = np.zeros(ids.size, bool); st[0] = True
            ustart.append(st)
            off += ids.size
        u.parent = np.concatenate(pars).astype(np.int32)
        ids = np.concatenate(idl)
        u.n = u.parent.size
        u.n_ctx = 0
        u.tokens = token[ids].astype(np.int32)
        r = radix_of[ids]
        starts = np.concatenate([[True], r[1:] != r[:-1]]) | np.concatenate(ustart)
        u.q2n = (np.cumsum(starts) - 1).astype(np.int32)
        u.qoff = np.concatenate([np.nonzero(starts)[0], [u.n]]).astype(np.int32)
        u.radix_ids = r[starts].astype(np.int32)
        u.mass_w = A.mass_weights(edge_mass[u.radix_ids], np.diff(u.qoff), "linear")
        units.append(u)
        pieces, rows = [], 0

    for b, e, o in zip(ub, ue, owner):
        if o != rank:
            continue
        b, e = int(b), int(e)
        pp = plan.parent_dfs[b:e].astype(np.int64) - b
        ids = d2n[b:e]
        if level == 2 and plan.depth[b] == 2:
            # bigram unit: the depth-1 ancestor rides along as a context row so every chain is complete
            a = int(plan.parent_dfs[b])
            pp = np.concatenate([[-1], pp + 1])
            pp[1] = 0
            ids = np.concatenate([[d2n[a]], ids])
        else:
            pp[plan.parent_dfs[b:e] < 0] = -1
        if rows and rows + ids.size > group_rows:
            flush()
        pieces.append((pp, ids))
        rows += ids.size
    flush()
    units.sort(key=lambda x: -x.n)
    total = int(plan.n)
    return units, counts, total, plan


# ----------------------------------------------------------------------------------------------------------
# the CPU arm: the oracle restatement of the reference's CPU path on the host cores
# ----------------------------------------------------------------------------------------------------------
def cpu_arm(units, cfg, budget_nodes, counts, steps=1, warmup=0):
    """Grouped forward + backward + per-query loss of the oracle on a bounded sample of units.
    Returns (nodes per second, cores, description)."""
    from oracle import pyoracle as O
    H, hd, V = cfg["heads"], cfg["head_dim"], cfg["vocab"]
    # launch groups from both ends of the size range in turn (largest, smallest, second largest, ...), as many as the budget holds
    by_size = sorted((u for u in units if u.n <= budget_nodes), key=lambda x: -x.n) or [min(units, key=lambda x: x.n)]
    order = []
    for i in range((len(by_size) + 1) // 2):
        order.append(by_size[i])
        if len(by_size) - 1 - i > i:
            order.append(by_size[len(by_size) - 1 - i])
    sample, tot = [], 0
    for u in order:
        if tot + u.n > budget_nodes and sample:
            continue
        sample.append(u)
        tot += u.n
        if tot >= budget_nodes:
            break
    rng = np.random.default_rng(0)
    data = []
    for u in sample:
        q, k, v, go = [rng.standard_normal((u.n, H * hd)).astype(np.float32) for _ in range(4)]
        data.append((u, q, k, v, go))

    def one_pass():
        # attention forward + backward only: what the GPU arm's end-to-end leg times as well
        for u, q, k, v, go in data:
            # local trees are in depth-first order, so parent < child holds
            out, w, w_off, _ = O.attn_fwd(u.parent, H, hd, q, k, v, grouped=True)
            roots = np.nonzero(u.parent < 0)[0]
            unit_off = np.concatenate([roots, [u.n]]).astype(np.int32)
            O.attn_bwd(u.parent, H, hd, q, k, v, w, w_off, go, unit_off=unit_off)
    for _ in range(warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    dt = (time.perf_counter() - t0) / steps
    return tot / dt, O.num_threads(), f"{len(sample)} launch groups of the same trie (sizes {min(u.n for u in sample)}..{max(u.n for u in sample)} rows, taken from both ends of the size range), {tot} positions, attention fwd+bwd (oracle, OpenMP)", dt


def run_reference(args):
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    units, counts, total, plan = build_units(args.workload, 0, args.gpus, lambda s: print(s, file=sys.stderr), group_rows=100_000)
    from oracle import pyoracle as O
    O.set_num_threads(os.cpu_count() or 1)      # torchrun pins OMP_NUM_THREADS=1; this arm may use every host core
    nps, cores, sample, dt = cpu_arm(units, cfg, args.cpu_nodes, counts, steps=max(1, args.steps), warmup=min(args.warmup, 1))
    line = {"impl": "reference", "metric": "trie_nodes_per_sec_attn_fwd_bwd", "value": nps, "unit": "nodes/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, cfg, total, args.gpus, int(plan.max_depth), np.bincount(plan.depth, minlength=2)[1:].tolist()),
            "cpu_baseline": {"value": nps, "unit": "nodes/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": nps, "unit": "nodes/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), file=RESULT_OUT, flush=True)


# ----------------------------------------------------------------------------------------------------------
# the GPU arm
# ----------------------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    import agpt_b200 as A

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    log = (lambda s: print(f"[bench r{rank}] {s}", file=sys.stderr, flush=True))
    cfg = WORKLOADS[args.workload]
    H, hd, V = cfg["heads"], cfg["head_dim"], cfg["vocab"]
    D = H * hd
    units, counts, total_nodes, gplan = build_units(args.workload, rank, world, log, args.single_unit, args.group_rows, device=local)
    n_rank = sum(u.n for u in units)
    n_max = max(u.n for u in units)
    log(f"{len(units)} launch groups, {n_rank} rows on this rank (largest {n_max}); {total_nodes} positions in the trie")

    plans = [A.WalkerPlan(u.parent, args.tile, local) for u in units]
    ws_bytes = max(p.workspace_bytes(D) for p in plans)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    # q k v dO resident for every row of the rank; when that exceeds 60 GB (the 126M-position configuration) all launch
    # groups read one set of buffers sized for the largest group instead (each group's rows are still far larger than L2)
    shared_inputs = 4 * n_rank * D * 4 > 60e9
    n_in = n_max if shared_inputs else n_rank
    big = [torch.randn((n_in, D), device=dev, generator=g) for _ in range(4)]
    kv_bytes = 4
    if args.kv == "bf16":        # the KV store holds bf16 rows (written once, outside the timed region, like a cache fill)
        big[1], big[2] = A.kv_store_write_bf16(big[1]), A.kv_store_write_bf16(big[2])
        kv_bytes = 2
    logits = torch.randn((n_in, V), device=dev, generator=g)
    out = torch.empty((n_max, D), device=dev); lse = torch.empty((n_max, H), device=dev)
    dq = torch.empty_like(out); dk = torch.empty_like(out); dv = torch.empty_like(out)
    dlogits = torch.empty((n_max, V), device=dev); loss = torch.empty(n_max, device=dev)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    c_off, c_tok, c_val = [torch.from_numpy(np.ascontiguousarray(c)).to(dev) for c in counts]
    meta = []
    row = 0
    for u in units:
        meta.append(dict(row=0 if shared_inputs else row, q2n=torch.from_numpy(u.q2n).to(dev), qoff=torch.from_numpy(u.qoff).to(dev),
                         rid=torch.from_numpy(u.radix_ids).to(dev), tok=torch.from_numpy(u.tokens).to(dev),
                         mw=torch.from_numpy(u.mass_w).to(dev)))
        row += u.n
    # gradient-sized buffer for the per-step all-reduce: the flat parameter vector of the config's model
    n_params = V * D + cfg["layers"] * (4 * (D * D + D) + 4 * D + 2 * 4 * D * D + 5 * D) + 2 * D + D * V + V
    grads = torch.zeros(n_params, device=dev)
    bwd_kernels = 0

    def step(timers=None):
        nonlocal bwd_kernels
        launches = 0
        for u, p, m in zip(units, plans, meta):
            sl = slice(m["row"], m["row"] + u.n)
            q, k, v, go = [t[sl] for t in big]
            if timers is not None:
                timers.append([torch.cuda.Event(enable_timing=True) for _ in range(4)])
                timers[-1][0].record()
            A.attn_forward(p, q, k, v, H, out=out[:u.n], lse=lse[:u.n])
            if timers is not None:
                timers[-1][1].record()
            A.attn_backward(p, q, k, v, out[:u.n], lse[:u.n], go, H, workspace=ws, dq=dq[:u.n], dk=dk[:u.n], dv=dv[:u.n])
            if timers is not None:
                timers[-1][2].record()
            check = A.lib().agpt_b200_loss_per_query(logits[sl].data_ptr(), m["q2n"].data_ptr(), m["qoff"].data_ptr(),
                                                     m["rid"].data_ptr(), m["tok"].data_ptr(), c_off.data_ptr(),
                                                     c_tok.data_ptr(), c_val.data_ptr(), m["mw"].data_ptr(),
                                                     dlogits.data_ptr(), loss.data_ptr(), u.n, V, 0.0, 1.0, 0,
                                                     torch.cuda.current_stream().cuda_stream)
            if check != 0:
                raise RuntimeError(A.lib().agpt_b200_last_error().decode())
            if timers is not None:
                timers[-1][3].record()
            launches += 2 + p.bwd_launches
        if world > 1:
            dist.all_reduce(grads)
        return launches

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    n_warm = args.warmup if args.profile else max(args.warmup, 3)
    for _ in range(n_warm):
        step()
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    launches = 0
    for _ in range(args.steps):
        launches += step()
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = total_nodes / (ms_per_step * 1e-3)

    # per-kernel durations (separate untimed-for-value pass, CUDA events on the launching stream)
    timers = []
    step(timers)
    torch.cuda.synchronize()
    t_fwd = sum(ev[0].elapsed_time(ev[1]) for ev in timers) * 1e-3
    t_bwd = sum(ev[1].elapsed_time(ev[2]) for ev in timers) * 1e-3
    t_loss = sum(ev[2].elapsed_time(ev[3]) for ev in timers) * 1e-3
    b_fwd = sum(p.algorithmic_bytes(D, H, kv_bytes)[0] for p in plans)
    b_bwd = sum(p.algorithmic_bytes(D, H, kv_bytes)[1] for p in plans)
    peak, peak_kind = measured_peak_gbs()
    # size-independent self-checks on the last group of the timing pass (outputs still in the buffers):
    # every query's weights sum to one, so sum_a dV_a == sum_i dO_i; and sum_i dq_i.q_i == sum_a dk_a.k_a
    u, m = units[-1], meta[-1]
    sl = slice(m["row"], m["row"] + u.n)
    qd, kd, god = big[0][sl].double(), big[1][sl].double(), big[3][sl].double()
    sv, sg = dv[:u.n].double().sum(0), god.sum(0)
    chk_dv = float((sv - sg).abs().max() / sg.abs().max())
    lhs, rhs = float((dq[:u.n].double() * qd).sum()), float((dk[:u.n].double() * kd).sum())
    chk_qk = abs(lhs - rhs) / max(abs(lhs), abs(rhs), 1e-30)
    selfcheck = {"sum_dv_vs_sum_dout_rel": chk_dv, "dq_dot_q_vs_dk_dot_k_rel": chk_qk,
                 "finite": bool(torch.isfinite(dq[:u.n]).all() and torch.isfinite(dk[:u.n]).all() and torch.isfinite(out[:u.n]).all())}
    del qd, kd, god
    # two byte models: touch-once (what must cross HBM; the roofline fraction) and the sibling-group-shared contract
    # model (every sibling group re-reads its ancestor chain; an algorithmic bandwidth that may exceed the peak
    # because the tile kernels share a chain among 64 depth-first neighbours and serve it from shared memory / L2)
    to_fwd, to_bwd = touch_once_bytes(n_rank, D, H, kv_bytes)
    ach_bwd, ach_fwd, ach_all = to_bwd / t_bwd / 1e9, to_fwd / t_fwd / 1e9, (to_fwd + to_bwd) / (t_fwd + t_bwd) / 1e9
    con_bwd, con_fwd, con_all = b_bwd / t_bwd / 1e9, b_fwd / t_fwd / 1e9, (b_fwd + b_bwd) / (t_fwd + t_bwd) / 1e9
    dram = DRAM_BYTES_PER_POSITION.get((D, args.kv))
    max_depth = int(gplan.max_depth)
    depth_hist = np.bincount(gplan.depth, minlength=2)[1:].tolist()

    # end to end: the host-buffer C-ABI call on a bounded subset of this rank's units; every rank runs its own sample
    # at the same time (each GPU has its own host link), time = max over ranks, rows = sum over ranks
    e2e = None
    if not args.no_e2e:
        budget = args.e2e_nodes
        chosen, tot = [], 0
        for u, p in zip(units, plans):
            if tot + u.n <= budget:
                chosen.append((u, p)); tot += u.n
        if not chosen:
            chosen, tot = [(units[-1], plans[-1])], units[-1].n
        numa = bind_to_gpu_numa_node(local)          # before the pinned buffers are allocated and first touched
        rng = np.random.default_rng(0)
        host = []
        for u, p in chosen:
            ins = [torch.from_numpy(rng.standard_normal((u.n, D), dtype=np.float32)).pin_memory() for _ in range(4)]
            outs = [torch.empty((u.n, D)).pin_memory(), torch.empty((u.n, H)).pin_memory()] + \
                   [torch.empty((u.n, D)).pin_memory() for _ in range(3)]
            host.append((u, p, [x.numpy() for x in ins], [x.numpy() for x in outs], ins, outs))
        for u, p, ins, outs, _, _ in host:                 # untimed: first call on a plan allocates its device arena
            A.attn_fwd_bwd_host(p, *ins, H, outs=outs)
        reps = 3
        sync_all()
        t0 = time.perf_counter()
        for _ in range(reps):
            for u, p, ins, outs, _, _ in host:
                A.attn_fwd_bwd_host(p, *ins, H, outs=outs)
        dt = (time.perf_counter() - t0) / reps
        tot_all = tot
        if world > 1:
            tmax = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            rows = torch.tensor([float(tot)], device=dev, dtype=torch.float64)
            dist.all_reduce(rows)
            dt, tot_all = float(tmax.item()), int(rows.item())
        e2e = {"value": tot_all / dt, "unit": "nodes/s", "h2d_bytes_per_step": int(tot_all * D * 4 * 4),
               "d2h_bytes_per_step": int(tot_all * (D * 4 * 4 + H * 4)),
               "sample": f"{len(chosen)} launch group(s) per rank, {tot_all} rows over {world} rank(s) ({tot} of {n_rank} on rank 0); "
                         "attention fwd+bwd through agpt_b200_attn_fwd_bwd_host, max time over ranks",
               "host_numa_rank0": numa}
        del host

    del big, logits, out, lse, dq, dk, dv, dlogits, loss, ws, plans, meta
    torch.cuda.empty_cache()

    # the attention-only microbenchmark (4M-node tree, 8 heads x 64) with both store types, as extra keys of the
    # default one-GPU line
    micro = None
    if args.micro and world == 1 and args.workload == "c2":
        micro = {kv: run_micro(kv, dev, log, peak) for kv in ("f32", "bf16")}

    # whole-epoch time of the trie-walk trainer on the same trie (all layers, loss, backward, one gradient
    # all-reduce and one optimizer step), every rank taking part
    epoch = None
    if args.epoch and not args.workload.startswith("micro"):
        epoch = run_epoch(args, cfg, rank, world, dev, log)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import pyoracle as O
        O.set_num_threads(os.cpu_count() or 1)
        small, _, _, _ = build_units(args.workload, 0, 1, lambda s: None, group_rows=100_000, device=local)
        nps, cores, sample, _ = cpu_arm(small, cfg, args.cpu_nodes, counts)
        cpu = {"value": nps, "unit": "nodes/s", "cores": cores, "kind": "port", "sample": sample}

    if rank == 0:
        line = {"metric": "trie_nodes_per_sec_attn_fwd_bwd", "value": value, "unit": "nodes/s", "n_gpus": world,
                "steps": args.steps, "warmup": n_warm, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(args, cfg, total_nodes, world, max_depth, depth_hist),
                "run": {"launch_groups_rank0": len(units), "group_rows": args.group_rows,
                        "inputs": "one buffer set shared by all launch groups" if shared_inputs else "resident for every row"},
                "roofline": {"bound": "hbm", "achieved": ach_bwd, "peak": peak, "unit": "GB/s", "frac": ach_bwd / peak,
                             "frac_contract": con_bwd / peak, "achieved_contract": con_bwd,
                             "traffic": (None if dram is None else dram[1] * n_rank),
                             "traffic_source": (None if dram is None else "ncu DRAM bytes per position of the reduced case of this workload x positions of this rank"),
                             "kernel": "attention backward tile kernel + dK/dV reduction", "peak_kind": f"of {peak_kind}",
                             "bytes_model": "touch-once (frac, achieved); sibling-group-shared contract model (frac_contract)",
                             "algorithmic_bytes_per_step": to_bwd, "contract_bytes_per_step": b_bwd, "seconds_per_step": t_bwd,
                             "fwd": {"achieved": ach_fwd, "frac": ach_fwd / peak, "frac_contract": con_fwd / peak,
                                     "algorithmic_bytes_per_step": to_fwd, "contract_bytes_per_step": b_fwd, "seconds_per_step": t_fwd,
                                     "traffic": (None if dram is None else dram[0] * n_rank)},
                             "fwd_bwd": {"achieved": ach_all, "frac": ach_all / peak, "frac_contract": con_all / peak},
                             "loss_seconds_per_step": t_loss},
                "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "micro": micro, "epoch": epoch,
                "selfcheck": selfcheck}
        print(json.dumps(line), file=RESULT_OUT, flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_micro(kv, dev, log, peak, steps=3, warmup=3, name="micro"):
    """Attention forward + backward on the microbenchmark tree (4M nodes, depth <= 64, geometric(0.35) children,
    8 heads x 64, Q/K/V/dO ~ N(0,1)), one launch over the whole tree; CUDA events per kernel."""
    import torch
    import agpt_b200 as A
    cfg = WORKLOADS[name]
    H, hd = cfg["heads"], cfg["head_dim"]
    D = H * hd
    parent = A.synth_tree(cfg["nodes"], cfg["depth"], 65, 0.35, 65, 75_000, 0)
    plan = A.WalkerPlan(parent, 64, dev.index)
    n = plan.n
    g = torch.Generator(device=dev).manual_seed(99)
    q, k, v, go = [torch.randn((n, D), device=dev, generator=g) for _ in range(4)]
    kvb = 4
    if kv == "bf16":
        k, v, kvb = A.kv_store_write_bf16(k), A.kv_store_write_bf16(v), 2
    out = torch.empty((n, D), device=dev); lse = torch.empty((n, H), device=dev)
    dq, dk, dv = [torch.empty((n, D), device=dev) for _ in range(3)]
    ws = torch.empty(plan.workspace_bytes(D), dtype=torch.uint8, device=dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    t_f = t_b = 0.0
    for i in range(warmup + steps):
        ev[0].record()
        A.attn_forward(plan, q, k, v, H, out=out, lse=lse)
        ev[1].record()
        A.attn_backward(plan, q, k, v, out, lse, go, H, workspace=ws, dq=dq, dk=dk, dv=dv)
        ev[2].record()
        torch.cuda.synchronize()
        if i >= warmup:
            t_f += ev[0].elapsed_time(ev[1]) * 1e-3 / steps
            t_b += ev[1].elapsed_time(ev[2]) * 1e-3 / steps
    to_f, to_b = touch_once_bytes(n, D, H, kvb)
    c_f, c_b = plan.algorithmic_bytes(D, H, kvb)
    res = {"nodes": n, "max_depth": int(plan.max_depth), "heads": H, "head_dim": hd, "kv_store": kv,
           "nodes_per_s": n / (t_f + t_b), "fwd_ms": t_f * 1e3, "bwd_ms": t_b * 1e3,
           "frac": {"fwd": to_f / t_f / 1e9 / peak, "bwd": to_b / t_b / 1e9 / peak, "fwd_bwd": (to_f + to_b) / (t_f + t_b) / 1e9 / peak},
           "frac_contract": {"fwd": c_f / t_f / 1e9 / peak, "bwd": c_b / t_b / 1e9 / peak, "fwd_bwd": (c_f + c_b) / (t_f + t_b) / 1e9 / peak},
           "finite": bool(torch.isfinite(dq).all() and torch.isfinite(dk).all() and torch.isfinite(dv).all())}
    log(f"{name} {kv}: fwd {t_f * 1e3:.1f} ms, bwd {t_b * 1e3:.1f} ms, {res['nodes_per_s'] / 1e6:.1f} M nodes/s")
    del q, k, v, go, out, lse, dq, dk, dv, ws, plan
    torch.cuda.empty_cache()
    return res


def run_epoch(args, cfg, rank, world, dev, log):
    """One timed epoch (after one untimed) of agpt_b200.trainer on the workload's trie with a seeded random-init
    model of the config's shape (d_ff = 4 d_model, N(0, 0.02) weights), rmsprop, linear mass weighting."""
    import torch
    import torch.distributed as dist
    import agpt_b200 as A
    from agpt_b200 import model_file as MF
    from agpt_b200 import trainer as T
    D = cfg["heads"] * cfg["head_dim"]
    corpus = A.synth_markov_corpus(cfg["chars"], cfg["vocab"], cfg["order"], 0, cfg.get("repeat_log2", 0))
    pm, pd = cfg.get("prune", (1, 4))
    trie = A.RadixTrie.build_gpu(corpus, cfg["depth"], 2, pm, pd, device=dev.index)
    mf = MF.random_init(D, cfg["heads"], cfg["layers"], cfg["vocab"], max(128, cfg["depth"]), seed=0)
    # a launch group keeps about 14 rows of d_model floats per position and layer for the backward pass: bound the
    # group so that this stays near 80 GB of the 180 GB
    group_rows = int(min(args.epoch_group_rows, 80e9 / (cfg["layers"] * D * 4 * 14)))
    groups, total = T.build_groups(trie, rank, world, group_rows, "linear", mf.seq_len, dev, level=2, unit_cap=group_rows)
    counts = [torch.from_numpy(np.ascontiguousarray(c)).to(dev) for c in (trie.cnt_off.astype(np.int32), trie.cnt_tok, trie.cnt_val)]
    model = T.TrieWalkModel(mf, dev)
    opt = T.make_optimizer("rmsprop", model, 3e-4, 0.999)
    times, losses = [], []
    for ep in range(2):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        ls, nq = T.train_epoch(model, groups, counts, opt, accumulate=True, world=world, bf16_store=(args.kv == "bf16"))
        torch.cuda.synchronize()
        t = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t.item()))
        losses.append(ls / max(nq, 1))
        log(f"epoch {ep + 1}: loss={losses[-1]:.6f} ({times[-1]:.2f} s, {len(groups)} chunks, {nq} nodes)")
    return {"seconds": times[-1], "positions_per_s": total / times[-1], "loss_first": losses[0], "loss_second": losses[-1],
            "model": f"d_model {D}, {cfg['layers']} layers, {cfg['heads']} heads x {cfg['head_dim']}, d_ff {4 * D}, vocab {cfg['vocab']}, fp32",
            "recipe": "rmsprop beta 0.999, lr 3e-4, linear mass weighting, one step per epoch (accumulate)", "kv_store": args.kv,
            "group_rows": group_rows, "partition": "bigram subtrees", "chunks_rank0": len(groups)}


# stdout carries the one JSON line and nothing else: what libraries print to file descriptor 1 (NCCL's version banner
# when the environment asks for it) goes to stderr with this program's own log
RESULT_OUT = sys.stdout


def main():
    global RESULT_OUT
    sys.stdout.flush()
    RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--tile", type=int, default=64)
    ap.add_argument("--kv", default="f32", choices=["f32", "bf16"], help="element type of the KV store")
    ap.add_argument("--cpu-nodes", type=int, default=400_000, help="rows in the CPU arm's sample")
    ap.add_argument("--e2e-nodes", type=int, default=4_000_000, help="rows in the host-buffer sample")
    ap.add_argument("--group-rows", type=int, default=4_000_000, help="rows per launch group (units are packed up to this)")
    ap.add_argument("--single-unit", action="store_true", help="one plan over the whole trie instead of per-subtree units")
    ap.add_argument("--profile", action="store_true", help="profiler capture mode: warm-up as given, no e2e, no CPU arm")
    ap.add_argument("--no-epoch", dest="epoch", action="store_false",
                    help="skip the whole-epoch timing of the trainer (all layers) on the same trie")
    ap.add_argument("--epoch-group-rows", type=int, default=4_000_000,
                    help="upper bound on the rows per launch group of the trainer epoch; also bounded by memory "
                         "(measured on c2: 1M rows 1.99 s, 2M 1.95 s, 4M 1.93 s)")
    ap.add_argument("--profile-epoch", action="store_true",
                    help="with --profile: keep the trainer epoch (to capture its dense-step kernels)")
    ap.add_argument("--no-micro", dest="micro", action="store_false",
                    help="skip the attention-only microbenchmark legs (4M-node tree, 8 x 64) of the default one-GPU line")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.profile:
        args.no_e2e = args.no_cpu = True
        args.epoch, args.micro = args.profile_epoch, False
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
