"""TEST INFRASTRUCTURE: pure-Python statement of the record a shard sends per row in the vocabulary-parallel
path (count, entries, statistics word - see fastertransformer_b200/vocab_parallel.py), used by the CPU tests of
the protocol."""
import numpy as np


def float_key(x):
    """Order-preserving uint32 image of float32 values (a < b  <=>  key(a) < key(b))."""
    b = np.asarray(x, dtype=np.float32).view(np.uint32)
    return np.where(b & 0x80000000, ~b, b | 0x80000000).astype(np.uint32)


def pack_record(values, k, cap, vocab_offset):
    """Record of one row of one shard: [count, cap entry slots, statistics word] as uint64, entries =
    (~key(value) << 32 | global column) for every column whose value reaches the shard's k-th largest value
    (whole tie class), sorted by value descending then column.  count = 2^64-1 if more than `cap` columns
    qualify.  The statistics word (soft-max pair of a top-p row) stays 0 for top-k rows."""
    values = np.asarray(values, dtype=np.float32)
    alive = np.flatnonzero(values > -np.finfo(np.float32).max)
    rec = np.zeros(2 + cap, dtype=np.uint64)
    if alive.size == 0:
        return rec
    order = alive[np.lexsort((alive, -values[alive].astype(np.float64)))]
    k_eff = min(k, order.size)
    kth = values[order[k_eff - 1]]
    m = int((values[order] >= kth).sum())
    if m > cap:
        rec[0] = np.uint64(0xFFFFFFFFFFFFFFFF)
        return rec
    rec[0] = m
    keys = (~float_key(values[order[:m]])).astype(np.uint64)
    rec[1:1 + m] = (keys << np.uint64(32)) | (order[:m].astype(np.uint64) + np.uint64(vocab_offset))
    return rec


def merge_records(records, vocab):
    """Union of the shards' records of one row as a dense row of length `vocab` (-inf where no shard sent
    the column), ready for any full-row selector."""
    row = np.full(vocab, -np.inf, dtype=np.float32)
    for rec in records:
        m = int(rec[0])
        ent = rec[1:1 + m]
        cols = (ent & np.uint64(0xFFFFFFFF)).astype(np.int64)
        keys = (~(ent >> np.uint64(32)).astype(np.uint32)).astype(np.uint32)
        bits = np.where(keys & 0x80000000, keys & 0x7FFFFFFF, ~keys).astype(np.uint32)
        row[cols] = bits.view(np.float32)
    return row
