"""B200 (sm_100a) implementation of BIDMach's Word2Vec skip-gram
negative-sampling minibatch path behind the reference's CUMACH interface.

``CUMACH``     the five native methods of edu.berkeley.bid.CUMACH for this path
``CUMACHSlice``  the vocabulary-slice forms of the update and scoring kernels
``Word2Vec``   host-side mirror of BIDMach.networks.Word2Vec (options, dobatch,
               evalbatch) above the C-ABI library
``Learner`` / ``ParLearner``  the minibatch schedule that drives it
``MatSource`` / ``FileSource``  minibatches from memory or from corpus files
``matio`` / ``modelio``  BIDMat matrix files, checkpoints, Google word2vec files
"""
from .cumach import CUMACH, CUMACHSlice, cuda_error_string  # noqa: F401
from .word2vec import Word2Vec  # noqa: F401
from .learner import Learner, ParLearner, MatSource  # noqa: F401
from .filesource import FileSource, FileSourceOpts  # noqa: F401
from . import matio, modelio  # noqa: F401
