"""Host-side mirror of ``BIDMach.networks.Word2Vec`` for the skip-gram
negative-sampling path (src/main/scala/BIDMach/networks/Word2Vec.scala).

The reference's host code is Scala; no JVM toolchain exists where this was
built, so the same interface -- option names and defaults, ``init`` /
``dobatch`` / ``evalbatch`` / ``wordMats`` / ``procPositives`` /
``procNegatives`` / ``evalPositives`` / ``evalNegatives`` / ``mergeModelFn`` --
is provided in Python above the C-ABI library.  PyTorch only supplies device
memory, streams and the process group; every computation happens in the CUDA
library, and nothing here works without it.
"""
from __future__ import annotations

import ctypes as C
import dataclasses

import numpy as np
import torch

from . import _lib, modelio
from .cumach import CUMACH, CUMACHSlice, cuda_error_string


@dataclasses.dataclass
class Opts:
    """``Word2Vec.Opts`` (Word2Vec.scala:574-591) with the inherited fields this
    path reads: ``dim`` (models/Model.scala:537), ``lrate``/``texp``
    (updaters/Grad.scala:242-243), ``vexp`` (updaters/ADAGrad.scala:158).
    Defaults are the reference's."""
    nskip: int = 5
    nneg: int = 5
    nreuse: int = 5
    vocabSize: int = 100000
    wexpt: float = 0.75
    wsample: float = 1e-4
    headlen: int = 10000
    iflip: bool = False
    eqPosNeg: bool = False
    maxArraySize: int = 2047 * 1024 * 1024
    nHeadTerms: int = 0
    nSlices: int = 1
    iSlice: int = 0
    dualMode: bool = False
    doHead: int = 1
    dim: int = 256
    lrate: float = 1.0
    texp: float = 0.5
    vexp: float = 0.5
    useGPU: bool = True
    seed: int = 0
    sortPermute: bool = False   # True: shuffle the pair list by sorting random keys (the reference's GPU branch)

    def to_c(self) -> _lib.W2VOpts:
        return _lib.W2VOpts(self.dim, self.nskip, self.nneg, self.nreuse, self.vocabSize,
                            self.wexpt, self.wsample, self.lrate, self.texp, self.vexp,
                            int(self.iflip), int(self.eqPosNeg), int(self.sortPermute), self.seed)


class _DevView:
    """A device buffer owned by the library, exposed through the CUDA array interface."""

    def __init__(self, ptr: int, n: int, typestr: str = "<i4"):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False),
                                         "version": 2}


def _view_i32(ptr: int, n: int, device) -> torch.Tensor:
    if n <= 0 or not ptr:
        return torch.empty(0, dtype=torch.int32, device=device)
    return torch.as_tensor(_DevView(ptr, n), device=device)


def _check(err: int, what: str):
    if err != 0:
        raise RuntimeError(f"{what} error " + cuda_error_string(err))


class Word2Vec:
    """SGNS model.  ``modelmats[0]`` is the context/embedding matrix (random
    init) and ``modelmats[1]`` the centre/negative matrix (zeros), both stored
    as ``[vocabSize, dim]`` fp32 CUDA tensors, i.e. the reference's column-major
    ``dim x vocabSize`` (Word2Vec.scala:113-117).

    With ``nSlices > 1`` the model holds one vocabulary slice (Word2Vec.scala:104-135, 665-672):
    the ``nHeadTerms`` most frequent words, which every slice has, followed by the words with
    ``id % nSlices == iSlice``; the matrices then have ``sliceRows()`` rows, minibatches still
    carry global ids, and every slice of a job sees every minibatch."""

    Opts = Opts

    def __init__(self, opts: Opts | None = None, device=None):
        self.opts = opts or Opts()
        if not self.opts.useGPU:
            raise RuntimeError("this build has no CPU path: useGPU must stay true")
        if self.opts.dualMode:
            raise NotImplementedError("dualMode keeps half of the model in host memory for the reference's "
                                      "CPU kernels; this build has no CPU path")
        if self.opts.nSlices < 1 or not 0 <= self.opts.iSlice < self.opts.nSlices or self.opts.nHeadTerms < 0:
            raise ValueError("need nSlices >= 1, 0 <= iSlice < nSlices, nHeadTerms >= 0")
        self.device = torch.device(device if device is not None else "cuda")
        self.modelmats: list[torch.Tensor] = []
        self.ncols = 0
        self._ctx = None
        self._copts = None
        self._batches = 0
        self._flat = None
        self._merge = None   # state of an averaging exchange in flight
        self._mc = 0         # NVLink multicast address of the model buffer (0: not in symmetric memory)
        self._symm = None
        self._tick = None

    def sliceRows(self) -> int:
        """Rows of each matrix: nHeadTerms + 1 + (vocabSize - nHeadTerms - 1) / nSlices
        (Word2Vec.scala:106), the whole vocabulary for one slice."""
        o = self.opts
        return int(_lib.load().w2v_slice_rows(o.vocabSize, o.nSlices, o.nHeadTerms))

    # -- life cycle ---------------------------------------------------------
    def init(self, ncols: int, refresh: bool = True):
        """Word2Vec.init (Word2Vec.scala:100-165): allocate both matrices and the
        per-minibatch work buffers for minibatches of ``ncols`` tokens."""
        o = self.opts
        lib = _lib.load()
        self.ncols = int(ncols)
        self._copts = o.to_c()
        with torch.cuda.device(self.device):
            if refresh or not self.modelmats:
                # both matrices in one buffer, so that one collective moves the whole model
                rows = self.sliceRows()
                self._flat = torch.empty(2, rows, o.dim, dtype=torch.float32, device=self.device)
                mm0, mm1 = self._flat[0], self._flat[1]
                shape = o.to_c()
                shape.vocabSize = rows     # the rows this model stores
                _check(lib.w2v_init_model(C.byref(shape), mm1.data_ptr(), mm0.data_ptr(),
                                          self._stream()), "w2v_init_model")
                self.modelmats = [mm0, mm1]
            ctx = C.c_void_p()
            err = lib.w2v_create(C.byref(self._copts), self.ncols, C.byref(ctx))
            if err:
                raise RuntimeError(f"w2v_create failed ({err}): unsupported options or out of memory")
            self._free_ctx()
            self._ctx = ctx
            if o.nSlices > 1:
                _check(lib.w2v_set_slice(ctx, o.iSlice, o.nSlices, o.nHeadTerms, o.doHead), "w2v_set_slice")
        return self

    def _free_ctx(self):
        if self._ctx is not None:
            _lib.load().w2v_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self._free_ctx()
        except Exception:
            pass

    def _stream(self) -> int:
        return int(torch.cuda.current_stream(self.device).cuda_stream)

    @staticmethod
    def _uniforms(u):
        if u is None:
            return None
        s = _lib.W2VUniforms(*(int(u[k].data_ptr()) if u.get(k) is not None else 0
                               for k in ("sample", "window", "permute", "negs")))
        return C.byref(s)

    # -- minibatch entry points --------------------------------------------
    def dobatch(self, gmats, ipass: int, pos: int, uniforms=None):
        """Word2Vec.dobatch (Word2Vec.scala:167-190).  ``gmats[0]`` is the device
        minibatch, int32 ``[ncols, 2]`` (word id, sentence id).  A minibatch of
        another length is skipped, as in the reference (:169)."""
        toks = gmats[0]
        if toks.shape[0] != self.ncols:
            return
        self._batches += 1
        with torch.cuda.device(self.device):
            _check(_lib.load().w2v_dobatch(self._ctx, toks.data_ptr(), self._uniforms(uniforms),
                                           self.modelmats[1].data_ptr(), self.modelmats[0].data_ptr(),
                                           int(pos), self._batches, self._stream()), "w2v_dobatch")
        if getattr(self, "_pending", None) is not None:
            self._launch_pending(after_pos=True)

    def evalbatch(self, gmats, ipass: int, pos: int, uniforms=None) -> float:
        """Word2Vec.evalbatch (Word2Vec.scala:192-212): mean log-likelihood score."""
        toks = gmats[0]
        if toks.shape[0] != self.ncols:
            return 0.0
        self.finishMerge()        # scores are taken on a model no exchange is writing to
        self._batches += 1
        score = C.c_double(0.0)
        with torch.cuda.device(self.device):
            _check(_lib.load().w2v_evalbatch(self._ctx, toks.data_ptr(), self._uniforms(uniforms),
                                             self.modelmats[1].data_ptr(), self.modelmats[0].data_ptr(),
                                             self._batches, C.byref(score), self._stream()),
                   "w2v_evalbatch")
        return score.value

    def dobatchg(self, mats, ipass: int, pos: int) -> int:
        """Model.dobatchg (models/Model.scala:350-354): the minibatch is still in
        host memory (numpy int32 ``[ncols, 2]`` or a CPU tensor); it is copied to
        the device inside the call.  Returns the number of positive pairs."""
        host = _host_i32(mats[0])
        if host.shape[0] != self.ncols:
            return 0
        self._batches += 1
        npairs = C.c_int64(0)
        with torch.cuda.device(self.device):
            _check(_lib.load().w2v_dobatch_host(self._ctx, host.ctypes.data,
                                                self.modelmats[1].data_ptr(), self.modelmats[0].data_ptr(),
                                                int(pos), self._batches, C.byref(npairs),
                                                self._stream()), "w2v_dobatch_host")
        if getattr(self, "_pending", None) is not None:
            self._launch_pending(after_pos=True)
        return npairs.value

    def evalbatchg(self, mats, ipass: int, pos: int) -> float:
        """Model.evalbatchg (models/Model.scala:356-365) for a host minibatch."""
        host = _host_i32(mats[0])
        if host.shape[0] != self.ncols:
            return 0.0
        self.finishMerge()
        self._batches += 1
        score = C.c_double(0.0)
        with torch.cuda.device(self.device):
            _check(_lib.load().w2v_evalbatch_host(self._ctx, host.ctypes.data,
                                                  self.modelmats[1].data_ptr(), self.modelmats[0].data_ptr(),
                                                  self._batches, C.byref(score), self._stream()),
                   "w2v_evalbatch_host")
        return score.value

    # -- the pieces, one reference method each ------------------------------
    def wordMats(self, gmats, ipass: int = 0, pos: int = 0, uniforms=None, batch_id: int = 0):
        """Word2Vec.wordMats (Word2Vec.scala:214-278).  Returns
        ``(words, lb, ub, trandwords, contextwords)`` as device tensors that alias
        the library's work buffers (valid until the next minibatch call):
        trandwords is ``[ngroups, nneg]`` and contextwords ``[ngroups, nreuse]``."""
        toks = gmats[0]
        lib = _lib.load()
        with torch.cuda.device(self.device):
            _check(lib.w2v_wordmats(self._ctx, toks.data_ptr(), self._uniforms(uniforms), batch_id,
                                    self._stream()), "w2v_wordmats")
        b = _lib.W2VBuffers()
        lib.w2v_buffers(self._ctx, C.byref(b))
        o, d = self.opts, self.device
        words = _view_i32(b.words, self.ncols, d)
        lb = _view_i32(b.lb, self.ncols, d)
        ub = _view_i32(b.ub, self.ncols, d)
        wa = _view_i32(b.WA, b.ngroups * o.nneg, d).view(-1, o.nneg)
        wb = _view_i32(b.WB, b.ngroups * o.nreuse, d).view(-1, o.nreuse)
        self.last_contexts = _view_i32(b.contexts, b.npairs, d)
        return words, lb, ub, wa, wb

    def procPositives(self, nskip, words, lbound, ubound, model1, model2, lrate, vexp):
        """Word2Vec.procPositives (Word2Vec.scala:366-383), GPU branch."""
        err = CUMACH.word2vecPos(model1.shape[1], words.numel(), nskip, words, lbound, ubound,
                                 model1, model2, lrate, vexp)
        _check(err, "CUMACH.word2vecPos")

    def procNegatives(self, nwa, nwb, wordsa, wordsb, modela, modelb, lrate, vexp):
        """Word2Vec.procNegatives (Word2Vec.scala:385-402), GPU branch."""
        err = CUMACH.word2vecNeg(modela.shape[1], wordsa.shape[0], nwa, nwb, wordsa, wordsb, modela,
                                 modelb, lrate, vexp)
        _check(err, "CUMACH.word2vecNeg")

    def evalPositives(self, nskip, words, lbound, ubound, model1, model2) -> float:
        """Word2Vec.evalPositives (Word2Vec.scala:469-489), GPU branch."""
        ret = torch.zeros(1, dtype=torch.float32, device=model1.device)
        err = CUMACH.word2vecEvalPos(model1.shape[1], words.numel(), nskip, words, lbound, ubound,
                                     model1, model2, ret)
        _check(err, "CUMACH.word2vecEvalPos")
        return float(ret.item())

    def evalNegatives(self, nwa, nwb, wordsa, wordsb, modela, modelb) -> float:
        """Word2Vec.evalNegatives (Word2Vec.scala:503-523), GPU branch."""
        ret = torch.zeros(1, dtype=torch.float32, device=modela.device)
        err = CUMACH.word2vecEvalNeg(modela.shape[1], wordsa.shape[0], nwa, nwb, wordsa, wordsb,
                                     modela, modelb, ret)
        _check(err, "CUMACH.word2vecEvalNeg")
        return float(ret.item())

    @staticmethod
    def mapIndx(indx: int, islice: int, nslices: int, nHead: int, maxCols: int, nrows: int, offset: int = 0):
        """Word2Vec.mapIndx (Word2Vec.scala:665-672): where word ``indx`` lives in slice ``islice``:
        (matrix block, element offset inside it, is it this slice's own word, is it a head word).
        The slices here keep all their rows in one matrix per side, i.e. ``maxCols`` at least
        ``sliceRows()``: the block is then ``offset`` and the element offset ``nrows`` times the
        row the slice kernels use."""
        newi = (indx - nHead) // nslices + nHead if indx >= nHead else indx
        m = newi // maxCols + offset
        ismine = indx >= nHead and indx % nslices == islice
        ishead = indx < nHead
        return m, nrows * (newi - m * maxCols), ismine, ishead

    # The slice forms take the two matrices of the slice (`modelmats`, rows as `sliceRows()` lays them
    # out) and the slice's number; slice count, head size and `doHead` come from the options.
    def procPositivesSlice(self, nskip, words, lbound, ubound, modelmats, lrate, vexp, islice):
        """Word2Vec.procPositivesSlice (Word2Vec.scala:404-433) on the device."""
        o = self.opts
        err = CUMACHSlice.word2vecPosSlice(modelmats[0].shape[1], words.numel(), nskip, words, lbound, ubound,
                                           modelmats[1], modelmats[0], lrate, vexp, islice, o.nSlices,
                                           o.nHeadTerms, o.doHead)
        _check(err, "word2vecPosSlice")

    def procNegativesSlice(self, nwa, nwb, wordsa, wordsb, modelmats, lrate, vexp, islice):
        """Word2Vec.procNegativesSlice (Word2Vec.scala:435-467) on the device."""
        o = self.opts
        err = CUMACHSlice.word2vecNegSlice(modelmats[0].shape[1], wordsa.shape[0], nwa, nwb, wordsa, wordsb,
                                           modelmats[1], modelmats[0], lrate, vexp, islice, o.nSlices,
                                           o.nHeadTerms, o.doHead)
        _check(err, "word2vecNegSlice")

    def evalPositivesSlice(self, nskip, words, lbound, ubound, modelmats, islice) -> float:
        """Word2Vec.evalPositivesSlice (Word2Vec.scala:491-501) on the device."""
        o = self.opts
        ret = torch.zeros(1, dtype=torch.float32, device=modelmats[0].device)
        err = CUMACHSlice.word2vecEvalPosSlice(modelmats[0].shape[1], words.numel(), nskip, words, lbound, ubound,
                                               modelmats[1], modelmats[0], ret, islice, o.nSlices, o.nHeadTerms)
        _check(err, "word2vecEvalPosSlice")
        return float(ret.item())

    def evalNegativesSlice(self, nwa, nwb, wordsa, wordsb, modelmats, islice) -> float:
        """Word2Vec.evalNegativesSlice (Word2Vec.scala:525-535) on the device."""
        o = self.opts
        ret = torch.zeros(1, dtype=torch.float32, device=modelmats[0].device)
        err = CUMACHSlice.word2vecEvalNegSlice(modelmats[0].shape[1], wordsa.shape[0], nwa, nwb, wordsa, wordsb,
                                               modelmats[1], modelmats[0], ret, islice, o.nSlices, o.nHeadTerms)
        _check(err, "word2vecEvalNegSlice")
        return float(ret.item())

    # -- multi-GPU ------------------------------------------------------------
    @staticmethod
    def mergeHeadLen(headlen: int, istep: int, vocab: int) -> int:
        """Rows of each matrix that sync number ``istep`` of the reference
        averages (Word2Vec.scala:548): all of them for ``istep == 0``, else the
        first ``max(headlen, headlen << trailingZeros(istep))`` (Int arithmetic:
        the shift count wraps at 32 and the product at 2^32), at most ``vocab``."""
        if istep <= 0:
            return vocab
        tz = (istep & -istep).bit_length() - 1
        shifted = (headlen << (tz & 31)) & 0xFFFFFFFF
        if shifted >= 1 << 31:
            shifted -= 1 << 32
        return min(vocab, max(headlen, shifted))

    def mergeModelFn(self, group=None, istep: int = 0):
        """Word2Vec.mergeModelFn (Word2Vec.scala:547-568): every replica ends up
        with the mean over the process group.  ``istep == 0`` (the default, and
        what the benchmark uses) averages the whole model, both matrices in one
        buffer, with one all-reduce (NCCL over NVLink when the group's backend is
        nccl) instead of the reference's host-driven peer copies; ``istep > 0``
        follows the reference's schedule and averages only the frequency-ranked
        head of each matrix (``mergeHeadLen`` rows).  Blocks the compute stream
        until the average is in."""
        import torch.distributed as dist
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return
        self.finishMerge()
        flat = getattr(self, "_flat", None)
        bufs = [flat] if flat is not None else self.modelmats
        if istep > 0:
            rows = self.mergeHeadLen(self.opts.headlen, istep, self.opts.vocabSize)
            if rows < self.opts.vocabSize:
                mats = flat if flat is not None else self.modelmats
                bufs = [mats[j][:rows] for j in range(2)]   # the head of a matrix is contiguous
        if getattr(self, "_mc", 0) and istep <= 0:
            # the model lives in symmetric memory: one averaging kernel per replica, fenced by two
            # one-element collectives (all replicas done updating / all slices written)
            self._inplace_average(group, 0)
            return
        avg = dist.ReduceOp.AVG if dist.get_backend(group) == "nccl" else None
        for m in bufs:
            if avg is not None:
                dist.all_reduce(m, op=avg, group=group)
            else:
                dist.all_reduce(m, op=dist.ReduceOp.SUM, group=group)
                m.mul_(1.0 / dist.get_world_size(group))

    def mergeHeadFn(self, group=None):
        """For a job whose replicas are vocabulary slices (``nSlices`` = replicas): the rows of the
        head (the first ``nHeadTerms`` of each matrix, which every slice holds and every slice
        updates from its own pairs) become their mean over the slices; the tail rows belong to one
        slice each and stay.  The reference leaves this step to its multi-node all-reduce outside
        the Word2Vec code; here it is one NCCL all-reduce per matrix (a contiguous block of rows)."""
        import torch.distributed as dist
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return
        self.finishMerge()
        rows = min(self.opts.nHeadTerms, self.modelmats[0].shape[0])
        if rows <= 0:
            return
        nccl = dist.get_backend(group) == "nccl"
        for m in self.modelmats:
            head = m[:rows]
            if nccl:
                dist.all_reduce(head, op=dist.ReduceOp.AVG, group=group)
            else:
                dist.all_reduce(head, op=dist.ReduceOp.SUM, group=group)
                head.mul_(1.0 / dist.get_world_size(group))

    # SMs the overlapped in-place average runs on, per replica count (24 beyond four): a replica
    # handles 1/world of the buffer, so fewer SMs keep up as the job grows.  Measured at two
    # replicas the step time hardly depends on the count between 24 and 64: fewer SMs lengthen the
    # exchange, more take them from the negative update beside it.
    EXCHANGE_BLOCKS = {2: 40, 3: 40, 4: 32}
    # replicas up to which the average uses peer loads and stores instead of the multicast
    # address (which moves a replica's own copy through the switch too: more bytes for few replicas)
    P2P_MAX_WORLD = 3

    def enableSymmetric(self, group=None) -> bool:
        """Moves the model into symmetric memory mapped on every replica's GPU through an NVLink
        multicast address, so that the exchange can run as w2v_nvls_average.  Collective: every
        rank of ``group`` calls it.  Returns False (and changes nothing) where the platform offers
        no multicast mapping; the exchange then stays with NCCL."""
        import torch.distributed as dist
        if getattr(self, "_mc", 0):
            return True
        if not dist.is_initialized() or dist.get_world_size(group) == 1 or self._flat is None:
            return False
        ok, hdl, buf = 1, None, None
        try:
            import torch.distributed._symmetric_memory as symm
            buf = symm.empty(self._flat.numel(), dtype=torch.float32, device=self.device)
            hdl = symm.rendezvous(buf, group=group if group is not None else dist.group.WORLD)
            if not int(getattr(hdl, "multicast_ptr", 0) or 0):
                ok = 0
        except Exception as e:   # no symmetric memory here: say why, stay with NCCL
            self._symm_error = repr(e)
            ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            return False
        buf.copy_(self._flat.view(-1))
        self._flat = buf.view(2, self.sliceRows(), self.opts.dim)
        self.modelmats = [self._flat[0], self._flat[1]]
        self._symm, self._mc = hdl, int(hdl.multicast_ptr)
        world = dist.get_world_size(group)
        self._peers = (C.c_void_p * world)(*[int(p) for p in hdl.buffer_ptrs])
        self._tick = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._pending = None
        return True

    def _inplace_average(self, group, blocks: int, kind: str | None = None):
        """Enqueues fence, averaging kernel, fence on the current stream.  ``kind``: "p2p" (peer
        loads and stores), "nvls" (multicast address), default by replica count."""
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        kind = kind or getattr(self, "exchangeKernel", None) or ("p2p" if world <= self.P2P_MAX_WORLD else "nvls")
        lib = _lib.load()
        dist.all_reduce(self._tick, group=group)     # every replica has finished its updates
        with torch.cuda.device(self.device):
            if kind == "p2p":
                _check(lib.w2v_p2p_average(self._peers, self._flat.numel(), rank, world, blocks,
                                           self._stream()), "w2v_p2p_average")
            else:
                _check(lib.w2v_nvls_average(self._mc, self._flat.numel(), rank, world, blocks,
                                            self._stream()), "w2v_nvls_average")
        dist.all_reduce(self._tick, group=group)     # every replica's slice has been written everywhere

    def reserveSMs(self, sms: int):
        """Keeps ``sms`` SMs out of the grid of the following minibatches' negative update (0 = use
        all), so that a kernel on another stream finds room."""
        with torch.cuda.device(self.device):
            _check(_lib.load().w2v_reserve_sms(self._ctx, int(sms)), "w2v_reserve_sms")

    def _launch_pending(self, after_pos: bool):
        """Starts the requested in-place average on the side stream: after the positive update of
        the minibatch just enqueued (so that it runs beside the negative update only, which loses
        nothing to it), or after everything enqueued so far."""
        group, blocks = self._pending
        self._pending = None
        if getattr(self, "_comm", None) is None:
            self._comm = torch.cuda.Stream(device=self.device, priority=-1)
        compute = torch.cuda.current_stream(self.device)
        if after_pos:
            with torch.cuda.device(self.device):
                _check(_lib.load().w2v_wait_pos(self._ctx, int(self._comm.cuda_stream)), "w2v_wait_pos")
        else:
            taken = torch.cuda.Event()
            taken.record(compute)
            self._comm.wait_event(taken)
        with torch.cuda.stream(self._comm):
            self._inplace_average(group, blocks)
            done = torch.cuda.Event()
            done.record(self._comm)
        self._merge = done
        self._merge_inplace = True

    def startMerge(self, group=None):
        """Overlapped form of mergeModelFn; training goes on while the exchange runs on a side
        stream, and ``finishMerge`` (called by the learner one minibatch later, or by the next
        start) makes the compute stream wait for it.

        With the model in symmetric memory the average is taken in place (w2v_nvls_average or
        w2v_p2p_average) on a few SMs beside the negative update of the next minibatch, which
        leaves them free; it starts when that minibatch's positive update has finished.  An element
        is read on all replicas, averaged and written back within microseconds, so it keeps every
        update made before and after that moment and loses only those that land in between.  Otherwise
        the model is snapshotted, the snapshot averaged with NCCL, and ``finishMerge`` adds
        ``average - snapshot`` to the live model (two extra model-sized buffers)."""
        import torch.distributed as dist
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return
        self.finishMerge()
        world = dist.get_world_size(group)
        if getattr(self, "_mc", 0):
            blocks = self.EXCHANGE_BLOCKS.get(world, 24)
            self._pending = (group, blocks)     # launched by the next minibatch call, or by finishMerge
            self.reserveSMs(blocks)
            return
        self._merge_inplace = False
        n = self._flat.numel()
        if getattr(self, "_snap", None) is None:
            self._snap = torch.empty_like(self._flat)
            self._avg = torch.empty_like(self._flat)
            self._shard = (torch.empty(n // world, dtype=torch.float32, device=self.device)
                           if n % world == 0 else None)
            self._comm = torch.cuda.Stream(device=self.device)
        compute = torch.cuda.current_stream(self.device)
        self._snap.copy_(self._flat)
        taken = torch.cuda.Event()
        taken.record(compute)
        nccl = dist.get_backend(group) == "nccl"   # other backends have no AVG: sum, then scale
        op = dist.ReduceOp.AVG if nccl else dist.ReduceOp.SUM
        with torch.cuda.stream(self._comm):
            self._comm.wait_event(taken)
            if self._shard is not None and nccl:
                # all-reduce as reduce-scatter + all-gather: both out of place, so the
                # snapshot survives without a second model-sized copy
                dist.reduce_scatter_tensor(self._shard, self._snap.view(-1), op=op, group=group)
                dist.all_gather_into_tensor(self._avg.view(-1), self._shard, group=group)
            else:
                self._avg.copy_(self._snap)
                dist.all_reduce(self._avg, op=op, group=group)
                if not nccl:
                    self._avg.mul_(1.0 / world)
            done = torch.cuda.Event()
            done.record(self._comm)
        self._merge = done

    def finishMerge(self, defer: bool = False):
        """Makes the compute stream wait for an exchange started by ``startMerge``.  ``defer``
        (in-place exchange only): not now but before the negative update of the next minibatch,
        so that an exchange that outlasts the negative update it ran beside finishes beside the
        next minibatch's preprocessing and positive update instead of stalling the stream."""
        if getattr(self, "_pending", None) is not None:
            self._launch_pending(after_pos=False)    # no minibatch came in between
        if getattr(self, "_deferred", None) is not None and not defer:
            # a wait handed to the next minibatch: take it now
            torch.cuda.current_stream(self.device).wait_event(self._deferred)
            if self._ctx is not None:     # the library must not keep an event that is about to go
                _lib.load().w2v_wait_before_neg(self._ctx, None)
            self._deferred = None
        if getattr(self, "_merge", None) is None:
            return
        compute = torch.cuda.current_stream(self.device)
        if getattr(self, "_merge_inplace", False):
            if defer:
                self._deferred = self._merge         # keeps the event alive until it has been waited for
                with torch.cuda.device(self.device):
                    _check(_lib.load().w2v_wait_before_neg(self._ctx, int(self._merge.cuda_event)),
                           "w2v_wait_before_neg")
            else:
                compute.wait_event(self._merge)
            self._merge = None
            self.reserveSMs(0)
            return
        compute.wait_event(self._merge)
        self._merge = None
        with torch.cuda.device(self.device):
            _check(_lib.load().w2v_apply_average(self._flat.data_ptr(), self._snap.data_ptr(),
                                                 self._avg.data_ptr(), self._flat.numel(),
                                                 self._stream()), "w2v_apply_average")

    # -- constructors and file formats of the companion object -----------------
    @staticmethod
    def learner(tokens, opts: "Opts | None" = None, batchSize: int = 1_000_000, lopts=None):
        """Word2Vec.learner (Word2Vec.scala:1222-1254): a single-GPU learner over an
        in-memory token matrix (int32 ``[ntokens, 2]``, the reference's
        ``learner(mat0)``) or, when ``tokens`` is a file-name pattern such as
        ``"data/train%05d.imat.lz4"``, over those files (``learner(fn1)``).
        Returns (learner, opts)."""
        from .learner import Learner
        opts = opts or Opts()
        return Learner(Word2Vec._source(tokens, batchSize, 0, 1), Word2Vec(opts), lopts), opts

    @staticmethod
    def _source(tokens, batchSize, rank, world):
        from .learner import MatSource
        if isinstance(tokens, str):
            from .filesource import FileSource, FileSourceOpts, simpleEnum
            return FileSource(FileSourceOpts(fnames=simpleEnum(tokens), batchSize=batchSize), rank, world)
        return MatSource(tokens, batchSize, rank, world)

    @staticmethod
    def learnPar(tokens, opts: "Opts | None" = None, batchSize: int = 1_000_000, lopts=None, group=None):
        """Word2Vec.learnPar (Word2Vec.scala:1312-1328): the data-parallel learner of
        this rank (one process per GPU, ``torch.distributed`` initialised) over a
        token matrix or a file-name pattern; the minibatches are dealt to the
        replicas in turn."""
        import torch.distributed as dist
        from .learner import ParLearner
        opts = opts or Opts()
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if opts.nSlices > 1:
            # replicas are vocabulary slices: slice = rank, every slice sees every minibatch and
            # draws the same samples (one minibatch's pairs are split over the slices)
            if opts.nSlices != world:
                raise ValueError("nSlices (%d) must equal the number of replicas (%d)" % (opts.nSlices, world))
            opts.iSlice = rank
            return ParLearner(Word2Vec._source(tokens, batchSize, 0, 1), Word2Vec(opts), lopts, group), opts
        opts.seed = opts.seed + 7919 * rank   # every replica draws its own samples
        return ParLearner(Word2Vec._source(tokens, batchSize, rank, world), Word2Vec(opts), lopts, group), opts

    def save(self, fname: str):
        """Model.save (models/Model.scala:245-263): ``options.json`` and
        ``modelmat00.lz4`` / ``modelmat01.lz4`` under ``fname``."""
        modelio.saveModel(fname, dataclasses.asdict(self.opts), self.modelmats)

    def delete(self, fname: str):
        """Model.delete (models/Model.scala:266-280): removes a checkpoint written by ``save``."""
        modelio.deleteModel(fname)

    def load(self, fname: str):
        """Model.load(fname, useJson = true) (models/Model.scala:282-315): the
        options of the checkpoint replace this model's, the matrices are copied
        onto the device."""
        o, mats = modelio.loadModel(fname)
        known = {f.name for f in dataclasses.fields(Opts)}
        for k, v in o.items():
            if k in known:
                setattr(self.opts, k, v)
        if len(mats) != 2 or mats[0].shape != (self.opts.vocabSize, self.opts.dim):
            raise ValueError("checkpoint holds %s, options say %d x %d" %
                             ([m.shape for m in mats], self.opts.vocabSize, self.opts.dim))
        if not getattr(self, "modelmats", None) or tuple(self.modelmats[0].shape) != mats[0].shape:
            self.init(getattr(self, "ncols", 0) or 1)
        for dst, src in zip(self.modelmats, mats):
            dst.copy_(torch.from_numpy(np.array(src, dtype=np.float32, order="C")))
        return self

    @staticmethod
    def predictor(model: "Word2Vec", tokens, batchSize: int | None = None):
        """Word2Vec.predictor (Word2Vec.scala:1282-1307): scores of a trained model on
        held-out tokens; call ``.predict(source)`` on the first element."""
        from .learner import Learner, MatSource
        src = MatSource(tokens, batchSize or model.ncols)
        return Learner(src, model), src

    saveGoogleW2V = staticmethod(modelio.saveGoogleW2V)
    readGoogleW2V = staticmethod(modelio.readGoogleW2V)


def _host_i32(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        if x.is_cuda:
            raise ValueError("dobatchg/evalbatchg take the minibatch in host memory")
        x = x.numpy()
    x = np.ascontiguousarray(x, dtype=np.int32)
    if x.ndim != 2 or x.shape[1] != 2:
        raise ValueError("minibatch must be int32 [ncols, 2] (word id, sentence id)")
    return x
