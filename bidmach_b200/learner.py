"""Minibatch schedule that drives the Word2Vec model: the part of
``BIDMach.Learner`` / ``ParLearner`` (src/main/scala/BIDMach/Learner.scala)
this path depends on.  Not a general training framework: only the loop, the
evaluation cadence and the multi-GPU exchange are mirrored.
"""
from __future__ import annotations

import dataclasses
import math
import time

import numpy as np

from .word2vec import Word2Vec


class MatSource:
    """In-memory data source: an int32 ``[ntokens, 2]`` array (word id, sentence
    id) handed out in minibatches of ``batchSize`` tokens, the last one short
    (datasources/MatSource.scala:78-91).  ``stride``/``offset`` give every rank
    of a data-parallel job its own minibatches, dealt round-robin as ParLearner
    deals them to its per-GPU threads (Learner.scala:638-651)."""

    def __init__(self, tokens: np.ndarray, batchSize: int, offset: int = 0, stride: int = 1):
        self.tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        self.batchSize = int(batchSize)
        self.offset, self.stride = offset, stride
        self.reset()

    def reset(self):
        self.k = self.offset

    @property
    def nbatches(self) -> int:
        return max(0, math.ceil((self._usable() - self.offset) / self.stride))

    def _usable(self) -> int:
        total = math.ceil(self.tokens.shape[0] / self.batchSize)
        # with several ranks every rank must see the same number of minibatches,
        # so the ragged tail of the deal is dropped
        return total if self.stride == 1 else (total // self.stride) * self.stride

    def hasNext(self) -> bool:
        return self.k < self._usable()

    def next(self):
        lo = self.k * self.batchSize
        self.k += self.stride
        return [self.tokens[lo: lo + self.batchSize]]

    def progress(self) -> float:
        return min(1.0, self.k * self.batchSize / max(1, self.tokens.shape[0]))


@dataclasses.dataclass
class LearnerOpts:
    """The fields of Learner.Opts / ParLearner.Opts this path reads
    (Learner.scala:1062-1081, 1152-1158), with the reference's defaults."""
    npasses: int = 2
    evalStep: int = 11
    updateAll: bool = False
    syncStep: int = 2
    overlapSync: bool = False   # not in the reference: exchange beside the next minibatch
    exchange: str = "auto"      # "nvls": average in place through the NVLink multicast mapping of the
                                # model buffer (w2v_nvls_average); "nccl": all-reduce; "auto": nvls where
                                # the platform has symmetric memory with multicast, else nccl
    headSync: bool = False      # the reference's schedule: syncs average a growing head of the vocabulary
    checkPointFile: str | None = None   # e.g. "ckpt/w2v%03d/": a checkpoint directory per number
    checkPointInterval: float = 0.0     # in passes over the data (Learner.scala:1074-1077)
    keepCheckPoints: int = 2
    nextCheckPoint: int = 0
    pstep: float = 0.01         # progress between two log lines (Learner.Opts.pstep)
    verbose: bool = False       # print the reference's progress lines
    logFile: str | None = None  # append one JSON object per progress line (pct, train, val, sec, words_per_s)


def _scala_mod(a: int, b: int) -> int:
    return int(math.fmod(a, b))


def _summary(scores, start: int) -> float:
    """Learner.scoreSummary without cumScore: the mean of the scores since ``start``."""
    part = scores[start:]
    return float(np.mean(part)) if part else float("nan")


class Learner:
    """Single-GPU loop, ``Learner.nextPass`` (Learner.scala:173-252): minibatch
    ``istep`` only scores when ``(istep - 1) % evalStep == 0`` or it is the last
    one of the pass (and not the first); every other minibatch trains, and the
    one with ``(istep - 1) % evalStep == 1`` is scored after it was trained on
    (the training score, ``trainlist``).  ``here`` advances by batchSize per
    minibatch and drives the learning-rate decay."""

    def __init__(self, datasource: MatSource, model: Word2Vec, opts: LearnerOpts | None = None):
        self.datasource, self.model = datasource, model
        self.opts = opts or LearnerOpts()
        self.reslist: list[float] = []
        self.samplist: list[int] = []
        self.trainlist: list[float] = []
        self.trainsamplist: list[int] = []
        self.here = 0
        self.ipass = 0
        self.nsamps = 0

    def init(self):
        self.model.init(self.datasource.batchSize)

    def _after_train_step(self, istep_global: int):
        pass

    def _after_minibatch(self):
        pass

    def train(self, do_init: bool = True):
        if do_init:
            self.init()
        self.here, self.ipass, self.nsamps = 0, 0, 0
        self.reslist, self.samplist = [], []
        self.trainlist, self.trainsamplist = [], []
        self._t0 = time.time()
        self._next_ckpt = self.opts.nextCheckPoint
        while self.ipass < self.opts.npasses:
            self.nextPass()
        self._before_wrapup()
        if self.opts.checkPointFile is not None and self._writes_checkpoints():   # Learner.wrapUp (Learner.scala:258-259)
            self.model.save(self.opts.checkPointFile % self._next_ckpt)
        return self

    def _before_wrapup(self):
        pass

    def _writes_checkpoints(self) -> bool:
        return True

    def loadCheckPoint(self, checkPointNumber: int = -1):
        """Learner.loadCheckPoint (Learner.scala:397-425): loads the given checkpoint, or
        the last one of the consecutive run found on disk, and continues the numbering."""
        import os
        o = self.opts
        lasti, found = -1, False
        while lasti < 100000:
            lasti += 1
            if os.path.exists((o.checkPointFile % lasti) + "options.json"):
                found = True
            elif found:
                break
        lasti -= 1
        if not found:
            print("loadCheckPoint: didnt find any checkpoint files")
            return False
        self.model.load(o.checkPointFile % (checkPointNumber if checkPointNumber >= 0 else lasti))
        o.nextCheckPoint = lasti + 1
        return True

    def nextPass(self):
        ds, o = self.datasource, self.opts
        ds.reset()
        istep = 0
        lastp, lasti, lastti = 0.0, len(self.reslist), len(self.trainlist)
        if o.verbose:
            print("pass=%2d" % self.ipass)
        while ds.hasNext():
            mats = ds.next()
            self.nsamps += mats[0].shape[0]
            self.here += ds.batchSize
            dsp = ds.progress()
            if _scala_mod(istep - 1, o.evalStep) == 0 or (istep > 0 and not ds.hasNext()):
                if o.updateAll:
                    self.model.dobatchg(mats, self.ipass, self.here)
                    self._after_train_step(istep)
                self.reslist.append(self.model.evalbatchg(mats, self.ipass, self.here))
                self.samplist.append(self.here)
            else:
                self.model.dobatchg(mats, self.ipass, self.here)
                self._after_train_step(istep)
                if _scala_mod(istep - 1, o.evalStep) == 1:      # Learner.scala:217-222
                    self.trainlist.append(self.model.evalbatchg(mats, self.ipass, self.here))
                    self.trainsamplist.append(self.here)
            self._after_minibatch()
            istep += 1
            if (o.verbose or o.logFile) and \
                    ((dsp > lastp + o.pstep and len(self.reslist) > lasti) or not ds.hasNext()):
                # the reference's line (Learner.scala:228-239) without its flop and memory columns
                lastp = (dsp - math.fmod(dsp, o.pstep)) if ds.hasNext() else 1.0
                secs = max(1e-9, time.time() - self._t0)
                tr, va = _summary(self.trainlist, lastti), _summary(self.reslist, lasti)
                if o.verbose:
                    print("%6.2f%%, train=%6.5f, val=%6.5f, sec=%2.0f, sam/s=%2.0f" % (
                        100.0 * lastp, tr, va, secs, self.nsamps / secs))
                if o.logFile:
                    import json
                    with open(o.logFile, "a") as f:
                        f.write(json.dumps({"pass": self.ipass, "pct": 100.0 * lastp,
                                            "train": None if math.isnan(tr) else tr,
                                            "val": None if math.isnan(va) else va, "sec": secs,
                                            "words_per_s": self.nsamps / secs, "here": self.here}) + "\n")
                lasti, lastti = len(self.reslist), len(self.trainlist)
            if o.checkPointFile is not None and \
                    self.ipass + dsp > o.checkPointInterval * (1 + self._next_ckpt - o.nextCheckPoint):
                # Learner.scala:242-249: save, then drop the checkpoint keepCheckPoints back
                old = self._next_ckpt - o.keepCheckPoints
                if self._writes_checkpoints():
                    self.model.save(o.checkPointFile % self._next_ckpt)
                    if o.keepCheckPoints > 0 and old >= 0:
                        self.model.delete(o.checkPointFile % old)
                self._next_ckpt += 1
        self.ipass += 1

    def predict(self, datasource: MatSource) -> list[float]:
        """Learner.predict (Learner.scala:322-391): score every full minibatch."""
        datasource.reset()
        out = []
        while datasource.hasNext():
            mats = datasource.next()
            if mats[0].shape[0] == self.model.ncols:
                out.append(self.model.evalbatchg(mats, 0, 0))
        return out


class ParLearner(Learner):
    """Data-parallel loop: one process per GPU, each with a full replica of both
    matrices and its own minibatches (or, when the model's ``nSlices`` > 1, each with one
    vocabulary slice and every minibatch: give every rank the same un-strided data source; the
    head rows are then averaged every ``syncStep`` training minibatches, ``Word2Vec.mergeHeadFn``); every ``syncStep`` training minibatches the
    replicas are averaged (ParLearner.syncmodels, Learner.scala:655, here one
    all-reduce per matrix, see Word2Vec.mergeModelFn).  Requires an initialised
    ``torch.distributed`` process group; rank 0's initial model is broadcast so
    that all replicas start equal (the reference's first full sync,
    Learner.scala:525)."""

    def __init__(self, datasource: MatSource, model: Word2Vec, opts: LearnerOpts | None = None,
                 group=None):
        super().__init__(datasource, model, opts)
        self.group = group
        self._since_sync = 0
        self._istep = 0          # ParLearner's istep: minibatches handed out over all replicas

    def init(self):
        import torch.distributed as dist
        super().init()
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            if self.opts.exchange in ("auto", "nvls") and not self.opts.headSync and not self._sliced() \
                    and dist.get_backend(self.group) == "nccl":
                if not self.model.enableSymmetric(self.group) and self.opts.exchange == "nvls":
                    raise RuntimeError("exchange='nvls': no symmetric memory with a multicast mapping here")
            src = dist.get_global_rank(self.group, 0) if self.group else 0
            if self._sliced():
                rows = self.model.opts.nHeadTerms     # slices share the head only
                for m in self.model.modelmats:
                    if rows > 0:
                        dist.broadcast(m[:rows], src=src, group=self.group)
            else:
                for m in self.model.modelmats:
                    dist.broadcast(m, src=src, group=self.group)

    def _world(self) -> int:
        import torch.distributed as dist
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def _after_minibatch(self):
        # Learner.scala:654-655: after every round of one minibatch per replica (scoring
        # rounds included), `istep += nthreads;
        # if ((istep/nthreads) % syncStep == 0) syncmodels(..., istep/syncStep, ...)`
        if not self.opts.headSync:
            return
        world = self._world()
        self._istep += world
        if (self._istep // world) % self.opts.syncStep == 0:
            self.model.mergeModelFn(self.group, self._istep // self.opts.syncStep)

    def _sliced(self) -> bool:
        o = getattr(self.model, "opts", None)
        return o is not None and getattr(o, "nSlices", 1) > 1

    def _after_train_step(self, istep_global: int):
        if self.opts.headSync:
            return
        self._since_sync += 1
        if self._sliced():
            # replicas are vocabulary slices: every one sees every minibatch, only the head is shared
            if self._since_sync >= self.opts.syncStep:
                self.model.mergeHeadFn(self.group)
                self._since_sync = 0
            return
        if self.opts.overlapSync:
            if self._since_sync == 1:
                self.model.finishMerge(defer=True)   # the exchange started beside this minibatch
            if self._since_sync >= self.opts.syncStep:
                self.model.startMerge(self.group)
                self._since_sync = 0
        elif self._since_sync >= self.opts.syncStep:
            self.model.mergeModelFn(self.group)
            self._since_sync = 0

    def _before_wrapup(self):
        # an exchange still in flight belongs to the model that the wrap-up checkpoint holds
        if self.opts.overlapSync:
            self.model.finishMerge()

    def _writes_checkpoints(self) -> bool:
        # the replicas share one checkpoint path: rank 0 writes and deletes, the others keep count
        import torch.distributed as dist
        return not dist.is_initialized() or dist.get_rank(self.group) == 0
