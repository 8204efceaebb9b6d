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
scaling) and both matrices are averaged over the replicas every
``--sync-every`` (8) minibatches, inside the timed region: in place through the
NVLink multicast mapping of the model buffer, beside the next minibatch, where
the platform offers one, else with an NCCL all-reduce.

Prints ONE JSON line (rank 0).  The timed region of `--steps` minibatches is
repeated `--repeats` times and the median region reported (`repeats` holds all
of them).  `value` is measured with the minibatches already in device memory;
`e2e` is the same loop through the host-buffer entry point (pinned host
minibatch -> device copy -> update -> pair count back).  `roofline` describes
the negative-update kernel: algorithmic bytes over its measured duration
against the measured HBM copy peak, the DRAM traffic of an ncu capture,
`compulsory_bytes` (every distinct row the launch names read once and written
once: a fraction that cannot exceed 1), and `memory_bound`: what the kernel's
atomic row additions, its row reads, and both together take on their own, on
the same columns (a probe library of its own, libw2vrowprobe.so).  `eval` is the scoring path
(configs[2]) on fixed random matrices, a shorter stretch of the same run.
With N > 1, `collective` describes the exchange: its kind, the bytes, what it
takes alone (CUDA events, max over ranks) and how many fell into the region.
`--impl reference` times the reference's own CPU kernels (compiled from its C
source into oracle/_ref) with all host cores on a bounded sample per step.

Other switches: `--mode eval` times the scoring path alone;
`--vocab / --tokens / --dim / --nneg / --wsample / --topics` change the
workload (configs[3] and [4]: `--topics 1000 --wsample 1e-4`,
`--topics 3000 --wsample 1e-4 --vocab 3000000 --nneg 10`); `--sort-permute`
shuffles the pair list by sorting random keys as the reference's GPU branch;
`--head-sync` selects the reference's head-only averaging schedule;
`--exchange nccl|nvls` and `--sync-mode blocking|overlap` the kind of exchange.
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the negative-update kernel on the
# default workload at the default rate 1e-3, i.e. with the folding period that the kernel derives
# from the hot word's share (6.49 GB read + 6.84 GB written; one-pass ncu capture of the
# full-size workload, six launches within 0.2 % of each other).
NEG_DRAM_TRAFFIC_BYTES = 13.33e9


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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
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


def cpu_threads():
    """Gives the CPU kernels every host core, whatever OMP_NUM_THREADS the launcher exported
    (torch.distributed.run sets it to 1), and returns (threads asked for, threads an OpenMP
    parallel region really runs with)."""
    from oracle import oracle as orc
    cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    return cores, orc.set_threads(cores)


def cpu_baseline(tokens, reps, warm=1):
    """The reference's CPU update kernels on a bounded sample of one minibatch: words/s."""
    cores, team = cpu_threads()
    kind = cpu_kind()
    orc, state = cpu_arm_setup(tokens)
    for _ in range(warm):
        cpu_arm_step(orc, state, kind, cores)
    t = [cpu_arm_step(orc, state, kind, cores) for _ in range(reps)]
    return {"value": CPU_SAMPLE / min(t), "unit": UNIT, "cores": team, "kind": kind,
            "sample_tokens": CPU_SAMPLE, "seconds_per_sample": t,
            "sample": f"first {CPU_SAMPLE} tokens of one 1M-token minibatch; positive + negative update "
                      f"kernels of the reference's BIDMach_CPUMACH.c split into {cores} chunks, run by an "
                      f"OpenMP team of {team} threads; best of {reps}; preprocessing untimed"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores, team = cpu_threads()
    kind = cpu_kind()
    pool = make_pool(0, 1)
    orc, state = cpu_arm_setup(pool[0])
    for _ in range(args.warmup):
        cpu_arm_step(orc, state, kind, cores)
    t = [cpu_arm_step(orc, state, kind, cores) for _ in range(args.steps)]
    total = float(np.sum(t))
    value = CPU_SAMPLE * args.steps / total
    sample = (f"first {CPU_SAMPLE} tokens of one 1M-token minibatch per step; positive + negative "
              f"update kernels of BIDMach_CPUMACH.c split into {cores} chunks, run by an OpenMP team of "
              f"{team} threads; preprocessing untimed")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config_dict(args),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": team, "kind": kind, "sample": sample,
                         "sample_tokens": CPU_SAMPLE},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# dram__bytes_read.sum per launch of the negative scoring kernel on the default workload (one-pass
# ncu capture of the full-size workload)
EVALNEG_DRAM_TRAFFIC_BYTES = 7.07e9


def config_dict(args, extra=None):
    w = WORKLOAD
    c = {"workload": "configs[1]: single-minibatch SGNS update, vocab 1M, dim 300, 1M-token "
                     "Zipf(1.07) minibatches, window 5, nneg 5, nreuse 5, no subsampling",
         "vocab": w["vocab"], "dim": w["dim"], "tokens_per_minibatch": w["ntokens"], "nskip": w["nskip"],
         "nneg": w["nneg"], "nreuse": w["nreuse"], "wsample": w["wsample"], "lrate": w["lrate"],
         "vexp": w["vexp"], "minibatch_pool": POOL,
         "parallelism": f"dp{args.gpus}: replicas, own minibatches, both matrices averaged over the replicas "
                        f"every {args.sync_every} minibatches"
                        + (" (head rows only, the reference's schedule)" if args.head_sync else "")
                        if args.gpus > 1 else "single GPU",
         "l2_policy": "inputs larger than L2: 2.4 GB of embedding rows gathered per Zipf draw; no flush"}
    if getattr(args, "slices", 1) > 1:
        c["slice"] = {"nSlices": args.slices, "iSlice": args.islice, "nHeadTerms": args.nhead}
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
    import ctypes as C

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
             sortPermute=args.sort_permute, nSlices=args.slices, iSlice=args.islice if args.slices > 1 else 0,
             nHeadTerms=args.nhead if args.slices > 1 else 0)
    model = Word2Vec(o, device=torch.device("cuda", local)).init(N)
    g = torch.Generator(device="cuda")

    def randomise_model():
        # configs[1] / configs[2]: both matrices U(-0.5, 0.5) / dim from a seed
        g.manual_seed(5)
        for m in model.modelmats:
            m.copy_((torch.rand(m.shape[0], w["dim"], device="cuda", generator=g) - 0.5) / w["dim"])

    # the exchange: in place through the NVLink multicast mapping where the platform has one
    exchange = "none"
    if world > 1:
        exchange = "nccl"
        if args.exchange in ("auto", "nvls") and not args.head_sync and model.enableSymmetric():
            exchange = "nvls"
        elif args.exchange == "nvls":
            raise SystemExit("--exchange nvls: no symmetric memory with a multicast mapping here (%s)"
                             % getattr(model, "_symm_error", "no multicast address"))
    if args.exchange_kernel:
        model.exchangeKernel = args.exchange_kernel
    if args.exchange_blocks:
        model.EXCHANGE_BLOCKS = {world: args.exchange_blocks}
    overlap = world > 1 and not args.head_sync and (
        args.sync_mode == "overlap" or (args.sync_mode == "auto" and exchange == "nvls"))
    randomise_model()
    if world > 1:
        for m in model.modelmats:
            dist.broadcast(m, src=0)

    pool = make_pool(rank, POOL)
    host = [torch.from_numpy(p).pin_memory() for p in pool]
    devt = [h.cuda() for h in host]
    stream = torch.cuda.current_stream()
    exch_events = []   # (start, end) events around every exchange of the current region

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def exchange_now(k):
        """The averaging exchange that follows minibatch k of a region (1-based)."""
        if args.head_sync:
            # the reference's schedule (Learner.scala:654-655, Word2Vec.scala:548): sync k averages
            # the first headlen << trailingZeros(k * world) rows of each matrix
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            model.mergeModelFn(None, k * world // args.sync_every)
            b.record(stream)
            exch_events.append((a, b))
        elif overlap:
            model.startMerge()          # runs beside the next minibatch; finishMerge follows it
            exch_events.append(None)
        else:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            model.mergeModelFn()
            b.record(stream)
            exch_events.append((a, b))

    def run_steps(nsteps, host_path, first_pos, mode, exchanges=True):
        """nsteps minibatches.  Exchanges follow the minibatches k with (nsteps - k) % sync_every == 0,
        so that a region holds ceil(nsteps / sync_every) of them, never fewer than its share."""
        pos = first_pos
        for s in range(1, nsteps + 1):
            pos += N
            b = (s - 1) % POOL
            if mode == "eval":
                if host_path:
                    model.evalbatchg([host[b].numpy()], 0, pos)
                else:
                    model.evalbatch([devt[b]], 0, pos)
                continue
            if host_path:
                model.dobatchg([host[b].numpy()], 0, pos)
            else:
                model.dobatch([devt[b]], 0, pos)
            if world > 1 and exchanges:
                if overlap:
                    model.finishMerge(defer=True)   # an exchange started beside this minibatch
                if (nsteps - s) % args.sync_every == 0:
                    exchange_now(s)
        return pos

    def timed(host_path, pos, mode, steps, warmup):
        """One warm-up stretch, then args.repeats regions of exactly `steps` minibatches, each
        bracketed by a device barrier; returns per-region ms (max over ranks) and bookkeeping
        of the median region."""
        pos = run_steps(warmup, host_path, pos, mode)
        if world > 1:
            model.finishMerge()
        regions = []
        for r in range(args.repeats):
            sync_all()
            lib.w2v_set_timing(model._ctx, 0 if host_path else 1)
            launches0 = lib.w2v_launch_count()
            del exch_events[:]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sampler.window_open()
            e0.record(stream)
            pos = run_steps(steps, host_path, pos, mode)
            if world > 1:
                model.finishMerge()   # an exchange still in flight belongs to the timed region
            e1.record(stream)
            sync_all()
            sampler.window_close()
            ms = e0.elapsed_time(e1)
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            tm = _lib.W2VTiming()
            lib.w2v_get_timing(model._ctx, tm)
            ex_ms = [a.elapsed_time(b) for (a, b) in [e for e in exch_events if e is not None]]
            regions.append({"ms": float(t.item()), "launches": lib.w2v_launch_count() - launches0,
                            "clocks": sampler.summary(), "timing": tm, "exchanges": len(exch_events),
                            "exchange_ms": ex_ms})
        order = sorted(range(len(regions)), key=lambda i: regions[i]["ms"])
        med = regions[order[len(order) // 2]]
        all_ms = [x["ms"] for x in regions]
        med["all_ms_per_step"] = [x / steps for x in all_ms]
        med["spread"] = (max(all_ms) - min(all_ms)) / med["ms"] if med["ms"] > 0 else None
        return med, pos

    probe = None

    def probe_bounds(reps=6):
        """The memory side of the negative kernels alone, on the workload's own columns:
        the update kernel's atomic row reductions with zeros (nothing else), the scoring
        kernel's row reads (nothing else), and both as the update kernel does them (a
        column's rows read, then zeros added to them).  ms per launch, CUDA events."""
        nonlocal probe
        path = os.path.join(os.path.dirname(_lib.LIB_PATH), "libw2vrowprobe.so")
        if not os.path.exists(path):
            return None
        if probe is None:
            probe = C.CDLL(path)
            probe.w2v_rowprobe.argtypes = [C.c_int] * 4 + [C.c_void_p] * 4 + [C.c_int, C.c_void_p]
        out = []
        for mode in (0, 1, 2):
            tot = 0.0
            for r in range(reps + 2):
                _, _, _, wa, wb = model.wordMats([devt[r % POOL]], batch_id=1000 + r)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                err = probe.w2v_rowprobe(w["dim"], wa.shape[0], w["nneg"], w["nreuse"], wa.data_ptr(), wb.data_ptr(),
                                         model.modelmats[1].data_ptr(), model.modelmats[0].data_ptr(), mode,
                                         model._stream())
                b.record(stream)
                torch.cuda.synchronize()
                if err:
                    return None
                if r >= 2:
                    tot += a.elapsed_time(b)
            out.append(tot / reps)
        return out

    def distinct_rows():
        """Distinct rows of A and of B that one minibatch's negative columns name (mean over the pool)."""
        na = nb_ = 0.0
        for k in range(POOL):
            _, _, _, wa, wb = model.wordMats([devt[k]], batch_id=2000 + k)
            na += float(torch.unique(wa).numel())
            nb_ += float(torch.unique(wb).numel())
        return na / POOL, nb_ / POOL

    def collective_alone(reps=3):
        """The exchange by itself, nothing else on the GPU: ms per exchange (max over ranks)."""
        out = []
        for _ in range(reps + 1):
            sync_all()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            model.mergeModelFn()
            b.record(stream)
            sync_all()
            t = torch.tensor([a.elapsed_time(b)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out.append(float(t.item()))
        return out[1:]

    peak, peak_kind = measured_peak_gbs()
    row = 4 * w["dim"]
    nr = (w["dim"] // 4 + 31) // 32
    default_shape = all(w[k] == DEFAULT_WORKLOAD[k] for k in ("vocab", "dim", "ntokens", "nneg", "nreuse", "nskip"))

    def eval_block(dev_r, e2e_r, steps, bounds):
        tm = dev_r["timing"]
        nb = max(1, tm.eval_batches)
        eg, ep = tm.eval_groups / nb, tm.eval_pairs / nb
        evalneg_ms, evalpos_ms = tm.evalneg_ms / nb, tm.evalpos_ms / nb
        nbytes = eg * (w["nneg"] + w["nreuse"]) * row
        achieved = nbytes / (evalneg_ms * 1e-3) / 1e9 if evalneg_ms > 0 else None
        traffic = EVALNEG_DRAM_TRAFFIC_BYTES if default_shape else None
        return {"metric": "SGNS eval (log-likelihood scoring) words/sec at vocab 1M dim 300",
                "workload": "configs[2]: scoring path, fixed random matrices, no update",
                "value": world * N * steps / (dev_r["ms"] * 1e-3), "unit": UNIT, "steps": steps,
                "ms_per_step": dev_r["ms"] / steps, "ms_per_step_all": dev_r["all_ms_per_step"],
                "e2e": {"value": world * N * steps / (e2e_r["ms"] * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": 8 * N, "d2h_bytes_per_step": 8},
                "gpu_launches": int(dev_r["launches"]),
                "phases": {"prep_ms": tm.prep_ms / nb, "permute_ms": tm.permute_ms / nb,
                           "evalpos_ms": evalpos_ms, "evalneg_ms": evalneg_ms,
                           "evalpos_algorithmic_gbs": (N + ep) * row / evalpos_ms / 1e6 if evalpos_ms > 0 else None},
                "roofline": {"bound": "hbm", "kernel": "neg_update_staged_kernel<%d,%d,%d,true>" % (
                                 w["nneg"], w["nreuse"], nr),
                             "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                             "frac": (achieved / peak) if achieved else None, "traffic": traffic,
                             "algorithmic_bytes_per_launch": nbytes, "avg_launch_ms": evalneg_ms,
                             "dram_frac": (traffic / (evalneg_ms * 1e-3) / 1e9 / peak)
                             if (traffic and evalneg_ms > 0) else None,
                             "memory_bound": ({"gather_only_ms": bounds[1],
                                               "kernel_over_gather_only": evalneg_ms / bounds[1]}
                                              if bounds else None)}}

    if args.mode == "exchange":
        # the exchange by itself at the workload's model size: NCCL, and where the model sits in
        # symmetric memory both in-place kernels over a range of SM counts (ms, max over ranks)
        if world < 2:
            raise SystemExit("--mode exchange needs --gpus >= 2")

        def time_of(fn, reps=5):
            ts = []
            for _ in range(reps + 1):
                sync_all()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                fn()
                b.record(stream)
                sync_all()
                t = torch.tensor([a.elapsed_time(b)], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ts.append(float(t.item()))
            return float(np.median(ts[1:]))

        flat = model._flat
        nbytes = 4 * flat.numel()
        out = {"mode": "exchange", "n_gpus": world, "bytes": nbytes, "symmetric_memory": exchange == "nvls",
               "nccl_allreduce_avg_ms": time_of(lambda: dist.all_reduce(flat, op=dist.ReduceOp.AVG)),
               "nccl_allreduce_sum_ms": time_of(lambda: dist.all_reduce(flat, op=dist.ReduceOp.SUM)),
               "fence_ms": None, "kernels": {}}
        if exchange == "nvls":
            out["fence_ms"] = time_of(lambda: dist.all_reduce(model._tick))
            s_ptr = model._stream()
            n = flat.numel()
            for kind in ("p2p", "nvls"):
                row = {}
                for blocks in (4, 8, 12, 16, 24, 32, 48, 64, 148):
                    if kind == "p2p":
                        fn = lambda: lib.w2v_p2p_average(model._peers, n, rank, world, blocks, s_ptr)
                    else:
                        fn = lambda: lib.w2v_nvls_average(model._mc, n, rank, world, blocks, s_ptr)
                    row[str(blocks)] = time_of(fn, reps=3)
                out["kernels"][kind] = row
            out["blocking_exchange_ms"] = time_of(lambda: model.mergeModelFn())
        sampler.stop()
        if rank == 0:
            print(json.dumps(out), flush=True)
        dist.destroy_process_group()
        return

    K = args.steps
    pos = 0
    if args.mode == "eval":
        dev_r, pos = timed(False, pos, "eval", K, args.warmup)
        e2e_r, pos = timed(True, pos, "eval", K, args.warmup)
        bounds = probe_bounds() if (rank == 0 and world == 1 and not args.no_probes and args.slices == 1) else None
        sampler.stop()
        if rank == 0:
            blk = eval_block(dev_r, e2e_r, K, bounds)
            line = {"metric": blk.pop("metric"), "value": blk["value"], "unit": UNIT, "n_gpus": world,
                    "steps": K, "warmup": args.warmup, "ms_per_step": blk["ms_per_step"],
                    "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                    "data": "synthetic",
                    "config": config_dict(args, extra={"workload": blk.pop("workload")}),
                    "e2e": blk["e2e"], "gpu_launches": blk["gpu_launches"], "phases": blk["phases"],
                    "roofline": blk["roofline"], "repeats": {"n": args.repeats,
                                                             "ms_per_step": blk["ms_per_step_all"],
                                                             "spread": dev_r["spread"]},
                    "clocks": dev_r["clocks"]}
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    dev_r, pos = timed(False, pos, "train", K, args.warmup)
    e2e_r, pos = timed(True, pos, "train", K, args.warmup)
    coll_alone = collective_alone() if world > 1 and not args.head_sync else None
    # the scoring path on fixed random matrices (configs[2]), a shorter stretch
    eval_blk = None
    if not args.no_eval:
        randomise_model()
        ke = max(4, min(K, 24))
        ev_dev, pos = timed(False, pos, "eval", ke, 3)
        ev_e2e, pos = timed(True, pos, "eval", ke, 3)
    bounds = probe_bounds() if (rank == 0 and world == 1 and not args.no_probes and args.slices == 1) else None
    rows_a, rows_b = distinct_rows() if (rank == 0 and not args.no_probes and args.slices == 1) else (0, 0)
    sampler.stop()
    if not args.no_eval and rank == 0:
        eval_blk = eval_block(ev_dev, ev_e2e, ke, bounds)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_dev, ms_e2e = dev_r["ms"], e2e_r["ms"]
    tm = dev_r["timing"]
    value = world * N * K / (ms_dev * 1e-3)
    e2e_value = world * N * K / (ms_e2e * 1e-3)
    nb = max(1, tm.train_batches)
    groups, pairs = tm.groups / nb, tm.pairs / nb
    neg_bytes = 2.0 * groups * (w["nneg"] + w["nreuse"]) * row
    neg_s = tm.neg_ms / nb * 1e-3
    pos_s = tm.pos_ms / nb * 1e-3
    achieved = neg_bytes / neg_s / 1e9 if neg_s > 0 else None
    # positive kernel, same accounting: (centres-with-pairs + pairs) rows read and written;
    # every token is kept in this workload, so centres ~ tokens
    pos_bytes = 2.0 * (N + pairs) * row
    # the DRAM traffic figure is an ncu capture of the default workload at the default rate; another
    # vocabulary, minibatch size or rate changes the L2 hit rate and the folding period
    traffic = NEG_DRAM_TRAFFIC_BYTES if (default_shape and w["lrate"] == DEFAULT_WORKLOAD["lrate"]) else None
    # what no kernel can avoid: every distinct row the launch names read once and written once
    compulsory = 2.0 * row * (rows_a + rows_b) if (rows_a + rows_b) > 0 else None
    roofline = {"bound": "hbm", "kernel": "neg_update_staged_kernel<%d,%d,%d,false>" % (
                    w["nneg"], w["nreuse"], nr), "achieved": achieved, "peak": peak,
                "peak_kind": peak_kind, "unit": "GB/s", "frac": (achieved / peak) if achieved else None,
                "traffic": traffic, "algorithmic_bytes_per_launch": neg_bytes,
                "avg_launch_ms": neg_s * 1e3,
                # the same fraction from the measured DRAM bytes instead of the algorithmic ones
                "dram_frac": (traffic / neg_s / 1e9 / peak) if (traffic and neg_s > 0) else None,
                # distinct rows read once + written once: at most 1 of peak by construction
                "compulsory_bytes": compulsory, "distinct_rows": {"A": rows_a, "B": rows_b},
                "compulsory_frac": (compulsory / neg_s / 1e9 / peak) if (compulsory and neg_s > 0) else None,
                "traffic_over_compulsory": (traffic / compulsory) if (traffic and compulsory) else None,
                # what the kernel's atomic row reductions take with nothing else in the kernel
                # (zeros added to the same rows), and what reading those rows takes: ms per launch
                # and what reading a column's rows and then adding zeros to them takes (the kernel's
                # whole memory side: its reductions find the rows in the L2, those of scatter_only do not)
                "memory_bound": ({"scatter_only_ms": bounds[0], "gather_only_ms": bounds[1],
                                  "gather_scatter_ms": bounds[2],
                                  "atomic_payload_gbs": neg_bytes / 2 / (bounds[0] * 1e-3) / 1e9,
                                  "kernel_over_scatter_only": neg_s * 1e3 / bounds[0],
                                  "kernel_over_gather_scatter": neg_s * 1e3 / bounds[2]} if bounds else None)}
    phases = {"prep_ms": tm.prep_ms / nb, "permute_ms": tm.permute_ms / nb, "pos_ms": tm.pos_ms / nb,
              "neg_ms": tm.neg_ms / nb, "pairs_per_step": pairs, "groups_per_step": groups,
              "pos_algorithmic_gbs": pos_bytes / pos_s / 1e9 if pos_s > 0 else None,
              "update_kernels_frac_of_peak": ((neg_bytes + pos_bytes) / (neg_s + pos_s) / 1e9 / peak)
              if neg_s + pos_s > 0 else None}

    collective = None
    if world > 1:
        nbytes = 4 * model._flat.numel()
        in_place = ("peer loads and stores on the replicas' symmetric buffers (w2v_p2p_average)"
                    if (args.exchange_kernel or ("p2p" if world <= model.P2P_MAX_WORLD else "nvls")) == "p2p"
                    else "multimem.ld_reduce/st over the NVLink multicast mapping (w2v_nvls_average)")
        collective = {"kind": ("in-place average kernel: " + in_place
                               if exchange == "nvls" else "ncclAllReduce(avg) via torch.distributed"),
                      "overlapped_with_next_minibatch": bool(overlap), "bytes": nbytes,
                      "sync_every": args.sync_every, "exchanges_in_region": dev_r["exchanges"],
                      "share_of_region": K / args.sync_every,
                      "in_region_ms": dev_r["exchange_ms"] or None}
        if coll_alone:
            t = float(np.median(coll_alone))
            collective.update({"alone_ms": t, "alone_all_ms": coll_alone,
                               "bus_gbs": 2.0 * (world - 1) / world * nbytes / (t * 1e-3) / 1e9,
                               "alg_gbs": nbytes / (t * 1e-3) / 1e9})
        if args.head_sync:
            collective["kind"] = "ncclAllReduce(avg) of the head rows (the reference's schedule)"

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(pool[0], reps=3)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": args.warmup,
        "ms_per_step": ms_dev / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(args),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 8 * N, "d2h_bytes_per_step": 8,
                "ms_per_step": ms_e2e / K, "ms_per_step_all": e2e_r["all_ms_per_step"],
                "spread": e2e_r["spread"]},
        "gpu_launches": int(dev_r["launches"]), "roofline": roofline, "cpu_baseline": cpu, "phases": phases,
        "repeats": {"n": args.repeats, "ms_per_step": dev_r["all_ms_per_step"], "spread": dev_r["spread"],
                    "reported": "median region"},
        "eval": eval_blk, "collective": collective,
        "clocks": dev_r["clocks"], "clocks_e2e": e2e_r["clocks"],
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=96)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=3,
                    help="timed regions of --steps minibatches each; the median region is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sync-every", type=int, default=8)
    ap.add_argument("--exchange", default="auto", choices=["auto", "nvls", "nccl"],
                    help="multi-GPU: average the model in place through the NVLink multicast mapping "
                         "(nvls; auto picks it where the platform has one) or with NCCL")
    ap.add_argument("--exchange-kernel", default=None, choices=["p2p", "nvls"],
                    help="force the in-place average's kernel (default: p2p up to 3 replicas, nvls beyond)")
    ap.add_argument("--exchange-blocks", type=int, default=None,
                    help="SMs the overlapped in-place average runs on (default by replica count)")
    ap.add_argument("--sync-mode", default="auto", choices=["auto", "overlap", "blocking"],
                    help="multi-GPU: run the exchange beside the next minibatch or block on it "
                         "(auto: overlap with nvls, blocking with nccl)")
    ap.add_argument("--head-sync", action="store_true",
                    help="average only the growing head of the vocabulary at each sync, as the reference's "
                         "mergeModelFn does, instead of the whole model")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-eval", action="store_true", help="skip the scoring stretch of the default run")
    ap.add_argument("--no-probes", action="store_true",
                    help="skip the row-traffic probes and the distinct-row count (profiling: keeps the launch list "
                         "to the minibatches)")
    ap.add_argument("--mode", default="train", choices=["train", "eval", "exchange"],
                    help="eval: time the scoring path (evalbatch) instead of the update path; exchange: time "
                         "the model exchange alone (NCCL, and the in-place kernels over a range of SM counts)")
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
    ap.add_argument("--slices", type=int, default=1,
                    help="single GPU: hold one vocabulary slice of this many (Word2Vec.Opts.nSlices) and work on "
                         "its share of every minibatch's pairs")
    ap.add_argument("--islice", type=int, default=0, help="which slice (Opts.iSlice)")
    ap.add_argument("--nhead", type=int, default=10000, help="head rows every slice holds (Opts.nHeadTerms)")
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
