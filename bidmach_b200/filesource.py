"""Minibatches from a sequence of corpus files, the part of
``BIDMach.datasources.FileSource`` (src/main/scala/BIDMach/datasources/FileSource.scala)
the Word2Vec scripts use: files ``fnames(n)`` for ``n`` in ``[nstart, nend)``, each a
2 x N int32 token matrix, cut into minibatches of ``batchSize`` tokens; a minibatch that
reaches the end of a file is completed from the head of the next one; ``lookahead``
threads read and decompress files ahead of the consumer.
"""
from __future__ import annotations

import dataclasses
import os
import threading
from typing import Callable

import numpy as np

from . import matio


def simpleEnum(fname: str, m: int = 1, i: int = 0) -> Callable[[int], str]:
    """FileSource.simpleEnum (FileSource.scala:380-387): ``n -> fname % (n*m + i)``."""
    return lambda n0: fname % (n0 * m + i)


def count_minibatches(sizes, batchSize: int) -> int:
    """How many minibatches ``FileSource.next`` cuts out of files of the given token
    counts (same walk as FileSource.scala:185-223: a minibatch spans at most two files)."""
    fileno, colno, k = 0, 0, 0
    while fileno < len(sizes):
        n = sizes[fileno]
        todo0 = min(batchSize, n - colno)
        todo1 = 0
        if todo0 < batchSize and fileno + 1 < len(sizes):
            todo1 = min(batchSize - todo0, sizes[fileno + 1])
        if todo1 == 0:
            if colno + todo0 == n:
                colno, fileno = 0, fileno + 1
            else:
                colno += todo0
        else:
            fileno, colno = fileno + 1, todo1
        k += 1
    return k


@dataclasses.dataclass
class FileSourceOpts:
    """FileSource.Opts (FileSource.scala:389-401) and DataSource.Opts.batchSize."""
    fnames: Callable[[int], str] | None = None
    batchSize: int = 10000
    lookahead: int = 2
    nstart: int = 0
    nend: int = 0            # 0: up to the first file that does not exist
    order: int = 0           # 0 = sequential, 1 = random order of the files (the last one stays last)
    throwMissing: bool = False
    seed: int = 0            # of the random file order


class FileSource:
    """``reset`` / ``hasNext`` / ``next`` / ``progress`` / ``close`` as the reference's
    class.  ``next`` returns ``[tokens]`` with tokens int32 ``[n, 2]`` (word id, sentence
    id), ``n == batchSize`` except for the tail of the last file.

    ``offset`` / ``stride`` deal the minibatches round-robin to the replicas of a
    data-parallel job, as ParLearner hands ``datasource.next`` to its threads in turn
    (Learner.scala:638-651): this source then returns minibatches ``offset``,
    ``offset + stride``, ... and stops when a whole round can no longer be dealt.
    """

    def __init__(self, opts: FileSourceOpts, offset: int = 0, stride: int = 1):
        if opts.fnames is None:
            raise ValueError("FileSourceOpts.fnames is not set")
        self.opts = opts
        self.offset, self.stride = offset, stride
        self.batchSize = opts.batchSize
        self._lock = threading.Condition()
        self._threads: list[threading.Thread] = []
        self._stop = False
        self._queue: dict[int, np.ndarray | None] = {}
        self._sizes: dict[int, int] = {}
        self.reset()

    # -- file bookkeeping ---------------------------------------------------
    def _exists(self, n: int) -> bool:
        return os.path.exists(self.opts.fnames(n))

    def reset(self):
        self.close()
        o = self.opts
        self.nstart, self.nend = o.nstart, o.nend
        if self.nend == 0:
            while self._exists(self.nend):
                self.nend += 1
        while self.nstart < self.nend and not self._exists(self.nstart):
            self.nstart += 1
        if self.nstart == self.nend:
            raise RuntimeError("Couldnt find any files")
        if o.order == 0:
            self._perm = lambda n: n
        else:
            # genperm (FileSource.scala:63-72): every file but the last in random order
            ii = np.random.default_rng(o.seed).permutation(self.nend - self.nstart - 1)
            self._perm = lambda n: n if n >= self.nend - 1 else self.nstart + int(ii[n - self.nstart])
        self.fileno, self.colno = self.nstart, 0
        self._fprogress = 0.0
        # with several replicas every one must see the same number of minibatches, so the
        # cut of the files into minibatches is planned from the file headers and the ragged
        # tail of the deal is dropped (as MatSource does)
        self._index = 0
        if self.stride > 1:
            sizes = [matio.peekShape(o.fnames(self._perm(n)))[1] for n in range(self.nstart, self.nend)]
            total = count_minibatches(sizes, self.batchSize)
            self._usable = (total // self.stride) * self.stride
        else:
            self._usable = None
        self._queue, self._sizes = {}, {}
        self._stop = False
        self._next_to_read = self.nstart
        for k in range(o.lookahead):
            t = threading.Thread(target=self._prefetch, daemon=True)
            t.start()
            self._threads.append(t)
        if self.stride > 1 or self.offset:
            self._skip(self.offset)

    def close(self):
        with self._lock:
            self._stop = True
            self._lock.notify_all()
        for t in self._threads:
            t.join()
        self._threads = []

    def _load(self, n: int) -> np.ndarray | None:
        fname = self.opts.fnames(self._perm(n))
        if not os.path.exists(fname):
            if n < self.nend and self.opts.throwMissing:
                raise RuntimeError("Missing file " + fname)
            return None
        return matio.loadTokens(fname)

    def _prefetch(self):
        while True:
            with self._lock:
                # stay at most lookahead + 1 files ahead of the consumer
                while not self._stop and (self._next_to_read >= self.nend or
                                          self._next_to_read > self.fileno + self.opts.lookahead + 1):
                    self._lock.wait(0.05)
                if self._stop:
                    return
                n = self._next_to_read
                self._next_to_read += 1
            try:
                mat = self._load(n)
            except Exception as e:            # handed to the consumer, which raises it
                mat = e
            with self._lock:
                self._queue[n] = mat
                self._lock.notify_all()

    def _file(self, n: int) -> np.ndarray:
        """Tokens of file number n (in reading order), waiting for a prefetcher if needed."""
        if self.opts.lookahead > 0:
            with self._lock:
                while n not in self._queue:
                    self._lock.wait(0.05)
                mat = self._queue[n]
        else:
            if n not in self._queue:
                self._queue[n] = self._load(n)
            mat = self._queue[n]
        if isinstance(mat, Exception):
            raise mat
        if mat is None:
            raise RuntimeError("Missing file %d" % n)
        return mat

    def _drop(self, n: int):
        with self._lock:
            self._queue.pop(n, None)
            self._lock.notify_all()

    # -- the reference's iteration (FileSource.scala:162-225) ----------------
    def hasNext(self) -> bool:
        if self._usable is None:
            return self.fileno < self.nend
        return self._index < self._usable

    def _take(self, copy: bool):
        cur = self._file(self.fileno)
        ncols = cur.shape[0]
        todo0 = min(self.batchSize, ncols - self.colno)
        todo1 = 0
        if todo0 < self.batchSize and self.fileno + 1 < self.nend:
            nxt = self._file(self.fileno + 1)
            todo1 = min(self.batchSize - todo0, nxt.shape[0])
        out = None
        if copy:
            if todo1 == 0:
                out = np.ascontiguousarray(cur[self.colno: self.colno + todo0])
            else:
                out = np.concatenate([cur[self.colno: self.colno + todo0], nxt[:todo1]])
        if todo1 == 0:
            if self.colno + todo0 == ncols:
                self._drop(self.fileno)
                self.colno, self.fileno = 0, self.fileno + 1
            else:
                self.colno += todo0
        else:
            self._drop(self.fileno)
            self.fileno, self.colno = self.fileno + 1, todo1
        self._fprogress = self.colno / max(1, ncols)
        return out

    def _skip(self, k: int):
        for _ in range(k):
            if self.fileno < self.nend:
                self._take(False)
                self._index += 1

    def next(self):
        out = self._take(True)
        self._index += 1
        if self.stride > 1:
            self._skip(self.stride - 1)
        return [out]

    def progress(self) -> float:
        return ((self.fileno - self.nstart) + self._fprogress) / max(1, self.nend - self.nstart)
