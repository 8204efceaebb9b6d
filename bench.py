#!/usr/bin/env python
"""Throughput of the Word2Vec SGNS minibatch path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one minibatch through the whole hot path: preprocessing
(subsampling, window bounds, pair list, permutation, negative ids), the
positive-pair update kernel and the negative-pair update kernel.  Workload
(BASELINE.json configs[1]): vocab 1M, dim 300 fp32, minibatches of 1M tokens
drawn i.i.d. from Zipf(1.07) over word ranks (seeded), window 5, 5 negatives,
nreuse 5, both matrices U(-0.5,0.5)/dim; frequent-word subsampling is switched
off (wsample=1 keeps every word), so every token yields pairs.

With N > 1 every rank runs the same workload on its own minibatches (weak
scaling) and both matrices are averaged with an all-reduce every
``--sync-every`` (8) minibatches, inside the timed region.

Prints ONE JSON line (rank 0).  `value` is measured with the minibatches
already in device memory; `e2e` is the same loop through the host-buffer entry
point (pinned host minibatch -> device copy -> update -> pair count back).
`roofline` describes the negative-update kernel: algorithmic bytes over its
measured duration against the measured HBM copy peak, the DRAM traffic of an
ncu capture, and `memory_bound`: what the kernel's atomic row additions and
its row reads take on their own, on the same columns (w2v_probe_rows).
`--impl reference` times the reference's own CPU kernels (compiled from its C
source into oracle/_ref) with all host cores on a bounded sample per step.

Other switches: `--mode eval` times the scoring path (configs[2]);
`--vocab / --tokens / --dim / --nneg / --wsample / --topics` change the
workload (configs[3] and [4]: `--topics 1000 --wsample 1e-4`,
`--topics 3000 --wsample 1e-4 --vocab 3000000 --nneg 10`); `--sort-permute`
shuffles the pair list by sorting random keys as the reference's GPU branch;
`--head-sync` / `--overlap-sync` select the reference's head-only averaging
schedule or an exchange overlapped with the next minibatch.
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

METRIC = "SGNS train words/sec at vocab 1M dim 300"
UNIT = "words/s"

WORKLOAD = dict(vocab=1_000_000, dim=300, ntokens=1_000_000, zipf_s=1.07, nskip=5, nneg=5, nreuse=5,
                lrate=1e-3, texp=0.5, vexp=0.5, wsample=1.0, doc_len=1000)
DEFAULT_WORKLOAD = dict(WORKLOAD)   # --vocab / --tokens / --nneg change WORKLOAD, not this
POOL = 4             # distinct minibatches per rank, cycled
CPU_SAMPLE = 500_000  # tokens of one minibatch the CPU arms process per step

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the negative-update
# kernel on this workload (6.48 GB read + 6.82 GB written), from a one-pass ncu
# capture of the full-size workload; see profiles/update_kernels_zipf_vocab1M_dim300.md.
NEG_DRAM_TRAFFIC_BYTES = 13.30e9


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index
        self.t0 = self.t1 = None

    def window_open(self):
        self.t0, self.t1 = time.monotonic(), None

    def window_close(self):
        self.t1 = time.monotonic()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [x.strip() for x in line.split(",")]))

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()

    def summary(self):
        """Clocks and throttle reasons of the samples inside the last window."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = list(self.rows)
        inside = [r for (t, r) in rows if self.t0 is None or (self.t0 <= t <= (self.t1 or t))]
        if not inside:  # region shorter than the sampling period: take the nearest sample
            inside = [r for (_, r) in rows[-1:]]
        for r in inside:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for k, nm in enumerate(names):
                if len(r) > 5 + k and r[5 + k].lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_pool(rank: int, n: int):
    from bidmach_b200.corpus import TopicCorpus, zipf_cdf, zipf_corpus
    w = WORKLOAD
    if w.get("topics"):
        # configs[3]/[4]: documents of a seeded topic model, 1000 tokens each
        tc = TopicCorpus(w["vocab"], w["topics"], w["zipf_s"], 0.1, w["doc_len"], seed=11)
        ndocs = w["ntokens"] // w["doc_len"]
        return [tc.tokens((rank * n + k) * ndocs, ndocs) for k in range(n)]
    cdf = zipf_cdf(w["vocab"], w["zipf_s"])
    return [zipf_corpus(w["vocab"], w["ntokens"], w["zipf_s"], seed=1000 * rank + k,
                        doc_len=w["doc_len"], cdf=cdf, first_doc=k * 1000) for k in range(n)]


# ---------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own C kernels on host cores
# ---------------------------------------------------------------------------

def cpu_arm_setup(tokens: np.ndarray, seed: int = 5):
    """Preprocess a CPU_SAMPLE-token prefix the CPU way and build host matrices."""
    from oracle import oracle as orc
    w = WORKLOAD
    rng = np.random.default_rng(seed)
    S = CPU_SAMPLE
    toks = np.ascontiguousarray(tokens[:S])
    words, lb, ub = orc.wordmats_bounds(toks, w["vocab"], w["nskip"], orc.salpha_of(w["wsample"], w["vocab"]),
                                        rng.random(S, dtype=np.float32), rng.random(S, dtype=np.float32))
    npairs = orc.count_pairs(words, lb, ub)
    WA, WB = orc.getnegs(words, lb, ub, w["nneg"], w["nreuse"], w["vocab"], orc.expt_of(0.75),
                         rng.random(npairs), rng.random(npairs // w["nreuse"] * w["nneg"] + 8, dtype=np.float32))
    mats = []
    for _ in range(2):
        m = np.empty((w["vocab"], w["dim"]), np.float32)
        rng.random(out=m, dtype=np.float32)
        m -= np.float32(0.5)
        m /= np.float32(w["dim"])
        mats.append(m)
    A, B = mats
    return orc, (words, lb, ub, WA, WB, A, B)


def cpu_arm_step(orc, state, kind: str, cores: int) -> float:
    """One bounded step of the CPU path: positive + negative update.  Seconds."""
    w = WORKLOAD
    words, lb, ub, WA, WB, A, B = state
    lr = np.float32(w["lrate"])
    t0 = time.perf_counter()
    orc.word2vecPos(w["dim"], len(words), w["nskip"], words, lb, ub, A, B, lr, w["vexp"], cores, kind)
    orc.word2vecNeg(w["dim"], WA.shape[0], w["nneg"], w["nreuse"], WA, WB, A, B, lr / w["nneg"],
                    w["vexp"], cores, kind)
    return time.perf_counter() - t0


def cpu_kind():
    from oracle import oracle as orc
    return "reference" if orc.have_reference() else "port"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    kind = cpu_kind()
    pool = make_pool(0, 1)
    orc, state = cpu_arm_setup(pool[0])
    for _ in range(args.warmup):
        cpu_arm_step(orc, state, kind, cores)
    t = [cpu_arm_step(orc, state, kind, cores) for _ in range(args.steps)]
    total = float(np.sum(t))
    value = CPU_SAMPLE * args.steps / total
    sample = (f"first {CPU_SAMPLE} tokens of one 1M-token minibatch per step; positive + negative "
              f"update kernels of BIDMach_CPUMACH.c, {cores} OpenMP threads; preprocessing untimed")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config_dict(args, extra={"cpu_sample_tokens": CPU_SAMPLE}),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# dram__bytes_read.sum per launch of the negative scoring kernel on the default workload
# (one-pass ncu capture; see profiles/scoring_kernels_zipf_vocab1M_dim300.md)
EVALNEG_DRAM_TRAFFIC_BYTES = 7.07e9


def eval_roofline(w, groups, row, evalneg_ms, bounds):
    """The negative scoring kernel against the HBM copy peak: rows read (algorithmic bytes)
    over its measured duration, the DRAM bytes of the ncu capture, and what reading the same
    rows and nothing else takes (ms per launch)."""
    peak, peak_kind = measured_peak_gbs()
    nbytes = groups * (w["nneg"] + w["nreuse"]) * row
    achieved = nbytes / (evalneg_ms * 1e-3) / 1e9 if evalneg_ms > 0 else None
    default_shape = all(w[k] == DEFAULT_WORKLOAD[k] for k in ("vocab", "dim", "ntokens", "nneg", "nreuse", "nskip"))
    traffic = EVALNEG_DRAM_TRAFFIC_BYTES if default_shape else None
    return {"bound": "hbm", "kernel": "neg_update_staged_kernel<%d,%d,%d,true>" % (
                w["nneg"], w["nreuse"], (w["dim"] // 4 + 31) // 32),
            "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
            "frac": (achieved / peak) if achieved else None, "traffic": traffic,
            "algorithmic_bytes_per_launch": nbytes, "avg_launch_ms": evalneg_ms,
            "dram_frac": (traffic / (evalneg_ms * 1e-3) / 1e9 / peak) if (traffic and evalneg_ms > 0) else None,
            "memory_bound": ({"gather_only_ms": bounds[1],
                              "kernel_over_gather_only": evalneg_ms / bounds[1]} if bounds else None)}


def config_dict(args, extra=None):
    w = WORKLOAD
    c = {"workload": "configs[1]: single-minibatch SGNS update, vocab 1M, dim 300, 1M-token "
                     "Zipf(1.07) minibatches, window 5, nneg 5, nreuse 5, no subsampling",
         "vocab": w["vocab"], "dim": w["dim"], "tokens_per_minibatch": w["ntokens"], "nskip": w["nskip"],
         "nneg": w["nneg"], "nreuse": w["nreuse"], "wsample": w["wsample"], "lrate": w["lrate"],
         "vexp": w["vexp"], "minibatch_pool": POOL,
         "parallelism": f"dp{args.gpus}: replicas, own minibatches, all-reduce(avg) of both matrices "
                        f"every {args.sync_every} minibatches"
                        + (" (overlapped with the next minibatch)" if args.overlap_sync else
                           " (head rows only, the reference's schedule)" if args.head_sync else " (blocking)")
                        if args.gpus > 1 else "single GPU",
         "l2_policy": "inputs larger than L2: 2.4 GB of embedding rows gathered per Zipf draw; no flush"}
    if w.get("topics"):
        c["workload"] = ("configs[3]/[4] shape: minibatches of %d-token documents from a seeded topic model "
                         "(%d topics, Zipf(%.2f) per topic, Dirichlet(0.1) mixtures), ids ranked by frequency"
                         % (w["doc_len"], w["topics"], w["zipf_s"]))
        c["topics"] = w["topics"]
    elif w["wsample"] != DEFAULT_WORKLOAD["wsample"] or w["vocab"] != DEFAULT_WORKLOAD["vocab"] \
            or w["nneg"] != DEFAULT_WORKLOAD["nneg"] or w["ntokens"] != DEFAULT_WORKLOAD["ntokens"] \
            or w["dim"] != DEFAULT_WORKLOAD["dim"]:
        c["workload"] = "configs[1] with overrides (see the fields below)"
    if extra:
        c.update(extra)
    return c


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist

    from bidmach_b200 import _lib, Word2Vec
    from bidmach_b200.word2vec import Opts

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for this path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _lib.load()
    w = WORKLOAD
    N = w["ntokens"]
    sampler = ClockSampler(local)   # runs for the whole job; each timed region reads its own window
    sampler.start()

    o = Opts(dim=w["dim"], vocabSize=w["vocab"], nskip=w["nskip"], nneg=w["nneg"], nreuse=w["nreuse"],
             lrate=w["lrate"], texp=w["texp"], vexp=w["vexp"], wsample=w["wsample"], seed=17 + rank,
             sortPermute=args.sort_permute)
    model = Word2Vec(o, device=torch.device("cuda", local)).init(N)
    # configs[1]: both matrices random
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    model.modelmats[1].copy_((torch.rand(w["vocab"], w["dim"], device="cuda", generator=g) - 0.5) / w["dim"])
    if world > 1:
        for m in model.modelmats:
            dist.broadcast(m, src=0)

    pool = make_pool(rank, POOL)
    host = [torch.from_numpy(p).pin_memory() for p in pool]
    devt = [h.cuda() for h in host]
    stream = torch.cuda.current_stream()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def run_steps(nsteps, host_path, first_pos):
        pos = first_pos
        for s in range(nsteps):
            pos += N
            if args.mode == "eval":
                if host_path:
                    model.evalbatchg([host[s % POOL].numpy()], 0, pos)
                else:
                    model.evalbatch([devt[s % POOL]], 0, pos)
                continue
            if host_path:
                model.dobatchg([host[s % POOL].numpy()], 0, pos)
            else:
                model.dobatch([devt[s % POOL]], 0, pos)
            if world > 1:
                if args.head_sync:
                    # the reference's schedule (Learner.scala:654-655, Word2Vec.scala:548): sync k
                    # averages the first headlen << trailingZeros(k * world) rows of each matrix
                    if (s + 1) % args.sync_every == 0:
                        model.mergeModelFn(None, (s + 1) * world // args.sync_every)
                elif not args.overlap_sync:
                    if (s + 1) % args.sync_every == 0:
                        model.mergeModelFn()
                else:   # the exchange runs beside the next minibatch and is folded in after it
                    if s % args.sync_every == 0:
                        model.finishMerge()
                    if (s + 1) % args.sync_every == 0:
                        model.startMerge()
        return pos

    def timed(host_path, pos):
        pos = run_steps(args.warmup, host_path, pos)
        sync_all()
        lib.w2v_set_timing(model._ctx, 0 if host_path else 1)
        launches0 = lib.w2v_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler.window_open()
        e0.record(stream)
        pos = run_steps(args.steps, host_path, pos)
        if world > 1:
            model.finishMerge()   # an exchange still in flight belongs to the timed region
        e1.record(stream)
        sync_all()
        sampler.window_close()
        clocks = sampler.summary()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), lib.w2v_launch_count() - launches0, clocks, pos

    def probe_bounds(reps=8):
        """The memory side of the negative kernels alone, on the workload's own columns:
        the update kernel's atomic row reductions with zeros (nothing else), and the
        scoring kernel's row reads (nothing else).  ms per launch, CUDA events."""
        out = []
        for mode in (0, 1):
            tot = 0.0
            for r in range(reps + 2):
                model.wordMats([devt[r % POOL]], batch_id=1000 + r)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                err = lib.w2v_probe_rows(model._ctx, model.modelmats[1].data_ptr(), model.modelmats[0].data_ptr(),
                                         mode, model._stream())
                b.record(stream)
                torch.cuda.synchronize()
                if err:
                    return None
                if r >= 2:
                    tot += a.elapsed_time(b)
            out.append(tot / reps)
        return out

    pos = 0
    ms_dev, launches, clocks, pos = timed(False, pos)
    tm = _lib.W2VTiming()
    lib.w2v_get_timing(model._ctx, tm)
    ms_e2e, _, clocks_e2e, pos = timed(True, pos)
    bounds = probe_bounds() if (rank == 0 and world == 1) else None
    sampler.stop()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    K = args.steps
    if args.mode == "eval":
        nb = max(1, tm.eval_batches)
        row = 4 * w["dim"]
        eg, ep = tm.eval_groups / nb, tm.eval_pairs / nb
        line = {"metric": "SGNS eval (log-likelihood scoring) words/sec at vocab 1M dim 300",
                "value": world * N * K / (ms_dev * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K,
                "warmup": args.warmup, "ms_per_step": ms_dev / K, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config_dict(args, extra={"workload": "configs[2]: scoring path, fixed random matrices"}),
                "e2e": {"value": world * N * K / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 8 * N,
                        "d2h_bytes_per_step": 8},
                "gpu_launches": int(launches),
                "phases": {"prep_ms": tm.prep_ms / nb, "permute_ms": tm.permute_ms / nb,
                           "evalpos_ms": tm.evalpos_ms / nb, "evalneg_ms": tm.evalneg_ms / nb,
                           "evalneg_algorithmic_gbs": eg * (w["nneg"] + w["nreuse"]) * row / (tm.evalneg_ms / nb) / 1e6,
                           "evalpos_algorithmic_gbs": (N + ep) * row / (tm.evalpos_ms / nb) / 1e6},
                "roofline": eval_roofline(w, eg, row, tm.evalneg_ms / nb, bounds),
                "clocks": clocks}
        print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    value = world * N * K / (ms_dev * 1e-3)
    e2e_value = world * N * K / (ms_e2e * 1e-3)
    peak, peak_kind = measured_peak_gbs()
    row = 4 * w["dim"]
    nb = max(1, tm.train_batches)
    groups, pairs = tm.groups / nb, tm.pairs / nb
    neg_bytes = 2.0 * groups * (w["nneg"] + w["nreuse"]) * row
    neg_s = tm.neg_ms / nb * 1e-3
    pos_s = tm.pos_ms / nb * 1e-3
    achieved = neg_bytes / neg_s / 1e9 if neg_s > 0 else None
    # positive kernel, same accounting: (centres-with-pairs + pairs) rows read and written;
    # every token is kept in this workload, so centres ~ tokens
    pos_bytes = 2.0 * (N + pairs) * row
    # the ncu capture was taken on the default workload; another vocabulary or minibatch size
    # changes the L2 hit rate, so no traffic figure is claimed for it
    default_shape = all(w[k] == DEFAULT_WORKLOAD[k] for k in ("vocab", "dim", "ntokens", "nneg", "nreuse", "nskip"))
    traffic = NEG_DRAM_TRAFFIC_BYTES if default_shape else None
    roofline = {"bound": "hbm", "kernel": "neg_update_staged_kernel<%d,%d,%d,false>" % (
                    w["nneg"], w["nreuse"], (w["dim"] // 4 + 31) // 32), "achieved": achieved, "peak": peak,
                "peak_kind": peak_kind, "unit": "GB/s", "frac": (achieved / peak) if achieved else None,
                "traffic": traffic, "algorithmic_bytes_per_launch": neg_bytes,
                "avg_launch_ms": neg_s * 1e3,
                # the same fraction from the measured DRAM bytes instead of the algorithmic ones
                "dram_frac": (traffic / neg_s / 1e9 / peak) if (traffic and neg_s > 0) else None,
                # what the kernel's atomic row reductions take with nothing else in the kernel
                # (zeros added to the same rows), and what reading those rows takes: ms per launch
                "memory_bound": ({"scatter_only_ms": bounds[0], "gather_only_ms": bounds[1],
                                  "atomic_payload_gbs": neg_bytes / 2 / (bounds[0] * 1e-3) / 1e9,
                                  "kernel_over_scatter_only": neg_s * 1e3 / bounds[0]} if bounds else None)}
    phases = {"prep_ms": tm.prep_ms / nb, "permute_ms": tm.permute_ms / nb, "pos_ms": tm.pos_ms / nb,
              "neg_ms": tm.neg_ms / nb, "pairs_per_step": pairs, "groups_per_step": groups,
              "pos_algorithmic_gbs": pos_bytes / pos_s / 1e9 if pos_s > 0 else None,
              "update_kernels_frac_of_peak": ((neg_bytes + pos_bytes) / (neg_s + pos_s) / 1e9 / peak)
              if neg_s + pos_s > 0 else None}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        kind = cpu_kind()
        orc, state = cpu_arm_setup(pool[0])
        cpu_arm_step(orc, state, kind, cores)
        reps = 3
        t = min(cpu_arm_step(orc, state, kind, cores) for _ in range(reps))
        cpu = {"value": CPU_SAMPLE / t, "unit": UNIT, "cores": cores, "kind": kind,
               "sample": f"first {CPU_SAMPLE} tokens of one minibatch, positive + negative update kernels "
                         f"of the reference's BIDMach_CPUMACH.c with {cores} OpenMP threads, best of {reps}; "
                         "preprocessing untimed"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": args.warmup,
        "ms_per_step": ms_dev / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(args),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 8 * N, "d2h_bytes_per_step": 8,
                "ms_per_step": ms_e2e / K},
        "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu, "phases": phases,
        "clocks": clocks, "clocks_e2e": clocks_e2e,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=96)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sync-every", type=int, default=8)
    ap.add_argument("--overlap-sync", action="store_true",
                    help="multi-GPU: run the averaging all-reduce beside the next minibatch (snapshot + "
                         "delayed correction) instead of blocking on it")
    ap.add_argument("--head-sync", action="store_true",
                    help="average only the growing head of the vocabulary at each sync, as the reference's "
                         "mergeModelFn does, instead of the whole model")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--mode", default="train", choices=["train", "eval"],
                    help="eval: time the scoring path (evalbatch) instead of the update path")
    ap.add_argument("--vocab", type=int, default=None, help="override the workload's vocabulary (profiling)")
    ap.add_argument("--tokens", type=int, default=None, help="override tokens per minibatch (profiling)")
    ap.add_argument("--nneg", type=int, default=None, help="override the number of negatives (configs[4] uses 10)")
    ap.add_argument("--dim", type=int, default=None, help="override the embedding dimension (a multiple of 4)")
    ap.add_argument("--lrate", type=float, default=None, help="override the learning rate (default 1e-3)")
    ap.add_argument("--wsample", type=float, default=None,
                    help="frequent-word subsampling (configs[3] and [4] use 1e-4; default: none)")
    ap.add_argument("--topics", type=int, default=None,
                    help="draw the minibatches from a topic-model corpus with this many topics "
                         "(configs[3]: 1000, configs[4]: 3000) instead of i.i.d. Zipf text")
    ap.add_argument("--sort-permute", action="store_true",
                    help="shuffle the pair list by sorting random keys (the reference's GPU branch) "
                         "instead of the keyed bijection")
    args = ap.parse_args()
    if args.vocab:
        WORKLOAD["vocab"] = args.vocab
    if args.tokens:
        WORKLOAD["ntokens"] = args.tokens
    if args.nneg:
        WORKLOAD["nneg"] = args.nneg
    if args.dim:
        WORKLOAD["dim"] = args.dim
    if args.lrate is not None:
        WORKLOAD["lrate"] = args.lrate
    if args.wsample is not None:
        WORKLOAD["wsample"] = args.wsample
    if args.topics:
        WORKLOAD["topics"] = args.topics
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
