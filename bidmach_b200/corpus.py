"""Seeded synthetic corpora in the reference's minibatch layout: int32
``[ntokens, 2]``, column 0 the word id, column 1 the sentence/document id.

Word ids are frequency ranks (id 0 the most frequent word), which is what the
reference's closed-form subsampling and negative sampling assume
(networks/Word2Vec.scala:150,221-225,265) and how its data preparation orders
the dictionary.  These corpora stand in for the 1-billion-word benchmark text
the reference's scripts train on, which is not redistributed here.
"""
from __future__ import annotations

import numpy as np


def zipf_cdf(vocab: int, s: float) -> np.ndarray:
    w = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    c = np.cumsum(w)
    return c / c[-1]


def zipf_corpus(vocab: int, ntokens: int, s: float = 1.0, seed: int = 0, doc_len: int = 1000,
                cdf: np.ndarray | None = None, first_doc: int = 0) -> np.ndarray:
    """Tokens drawn i.i.d. from Zipf(s) over word ranks; a new sentence id every
    ``doc_len`` tokens."""
    rng = np.random.Generator(np.random.Philox(seed))
    if cdf is None:
        cdf = zipf_cdf(vocab, s)
    ids = np.searchsorted(cdf, rng.random(ntokens), side="right").astype(np.int32)
    np.minimum(ids, vocab - 1, out=ids)
    out = np.empty((ntokens, 2), np.int32)
    out[:, 0] = ids
    out[:, 1] = first_doc + np.arange(ntokens, dtype=np.int64) // doc_len
    return out


class TopicCorpus:
    """Structured corpus: ``ntopics`` topics, each a Zipf(s) distribution over its
    own permutation of the vocabulary; documents of ``doc_len`` tokens whose topic
    mixture is Dirichlet(alpha); word ids re-ranked by global expected frequency.

    The per-topic permutations are affine maps ``r -> (a_t * r + b_t) mod vocab``
    with ``a_t`` coprime to ``vocab`` (a table of explicit permutations would take
    ntopics * vocab * 4 bytes: 4 GB at 1000 x 1M).  Minibatches are generated on
    demand from (seed, document number), so a stream of any length can be cut
    into per-rank shards without materialising it.
    """

    def __init__(self, vocab: int, ntopics: int, s: float = 1.07, alpha: float = 0.1,
                 doc_len: int = 1000, seed: int = 0, rank_sample_docs: int = 20000):
        self.vocab, self.ntopics, self.s, self.alpha = vocab, ntopics, s, alpha
        self.doc_len, self.seed = doc_len, seed
        self.cdf = zipf_cdf(vocab, s)
        rng = np.random.Generator(np.random.Philox(seed))
        a = rng.integers(1, vocab, size=ntopics, dtype=np.int64)
        for t in range(ntopics):
            while np.gcd(int(a[t]), vocab) != 1:
                a[t] = (a[t] + 1) % vocab or 1
        self.a = a
        self.b = rng.integers(0, vocab, size=ntopics, dtype=np.int64)
        # frequency ranks: expected counts are estimated once from a fixed seeded
        # sample of documents, then ids are renumbered by descending count
        raw = self._raw_docs(np.arange(rank_sample_docs, dtype=np.int64) + (1 << 40))
        counts = np.bincount(raw.ravel(), minlength=vocab)
        order = np.argsort(-counts, kind="stable")
        self.rank_of = np.empty(vocab, np.int32)
        self.rank_of[order] = np.arange(vocab, dtype=np.int32)

    def _raw_docs(self, doc_ids: np.ndarray) -> np.ndarray:
        out = np.empty((len(doc_ids), self.doc_len), np.int64)
        for k, d in enumerate(doc_ids):
            rng = np.random.Generator(np.random.Philox(key=[self.seed, int(d)]))
            theta = rng.dirichlet(np.full(self.ntopics, self.alpha))
            z = rng.choice(self.ntopics, size=self.doc_len, p=theta)
            r = np.searchsorted(self.cdf, rng.random(self.doc_len), side="right")
            np.minimum(r, self.vocab - 1, out=r)
            out[k] = (self.a[z] * r + self.b[z]) % self.vocab
        return out

    def tokens(self, first_doc: int, ndocs: int) -> np.ndarray:
        """Documents ``first_doc .. first_doc+ndocs-1`` as int32 ``[ndocs*doc_len, 2]``."""
        docs = np.arange(first_doc, first_doc + ndocs, dtype=np.int64)
        raw = self._raw_docs(docs)
        out = np.empty((ndocs * self.doc_len, 2), np.int32)
        out[:, 0] = self.rank_of[raw.ravel()]
        out[:, 1] = np.repeat(docs, self.doc_len).astype(np.int32)
        return out
