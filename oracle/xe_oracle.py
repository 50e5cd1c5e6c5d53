"""CPU restatement (numpy) of the shared-model cost of the reference's offline study
(scripts/llama-3-8b/experiment_2_1.py in the Checkers tree).  Test infrastructure only: the product path is
Context.shared_model_cost (CUDA).  Pinned by tests/golden/xe_golden.json, written from the reference's functions.

  build_model   counts -> quantised counts summing to a power-of-two scale   (:52-75)
  merge         vocabularies and counts of several tensors -> the group's      (:217-235)
  cost          sum over the group's tensors of count * log2(scale / norm)     (:238-270, 273-330)
"""
import numpy as np

PRECISION = 14


def build_model(counts):
    n_vocab = len(counts)
    p = max(PRECISION, int(np.ceil(np.log2(max(n_vocab, 2)))) + 1)
    scale = 1 << p
    total = int(counts.sum())
    norm = np.floor(counts * (scale / total)).astype(np.int64)
    norm = np.maximum(norm, 1)
    norm[np.argmax(counts)] += scale - int(norm.sum())
    return np.maximum(norm, 1), scale


def vocabulary(symbols):
    return np.unique(symbols, return_counts=True)


def merge(vocab_list, counts_list):
    all_v = np.concatenate([v.astype(np.int64) for v in vocab_list])
    all_c = np.concatenate([c.astype(np.int64) for c in counts_list])
    order = np.argsort(all_v, kind="stable")
    sv, sc = all_v[order], all_c[order]
    change = np.concatenate([[True], sv[1:] != sv[:-1]])
    return sv[change].astype(np.uint32), np.add.reduceat(sc, np.where(change)[0]).astype(np.int64)


def shared_model_cost(symbol_arrays):
    """(stream bytes, vocabulary size) of the tensors coded under one model over their 32-bit symbols."""
    summaries = [vocabulary(s) for s in symbol_arrays if s.size]
    if not summaries:
        return 0.0, 0
    cv, cc = merge([v for v, _ in summaries], [c for _, c in summaries])
    norm, scale = build_model(cc)
    normf = norm.astype(np.float64)
    bits = 0.0
    for v, c in summaries:
        idx = np.searchsorted(cv.astype(np.int64), v.astype(np.int64))
        bits += float(np.sum(c.astype(np.float64) * np.log2(scale / normf[idx])))
    return bits / 8.0, int(cv.size)
