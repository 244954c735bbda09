"""Buffer pool -- the role of src/pool.js in the reference.

Buffers are recycled by power-of-two size class and storage mode
(src/pool.js:8-13, 26-49).  The allocator behind it is injectable so the
bucketing logic can be exercised without a device.
"""
from . import device

_sharedPool = {}
_privatePool = {}
_hits = 0
_misses = 0
_totalAllocated = 0
_allocFn = None  # defaults to device.alloc


def setAllocFn(fn):
    global _allocFn
    _allocFn = fn


def bucketSize(nbytes):
    """Next power of two, minimum 256 (src/pool.js:8-13)."""
    if nbytes <= 256:
        return 256
    s = 1
    while s < nbytes:
        s <<= 1
    return s


def poolAlloc(nbytes, mode=device.SHARED):
    global _hits, _misses, _totalAllocated
    bucket = bucketSize(nbytes)
    pool = _privatePool if mode == device.PRIVATE else _sharedPool
    bin_ = pool.get(bucket)
    if bin_:
        _hits += 1
        return bin_.pop()["buffer"]
    _misses += 1
    _totalAllocated += bucket
    return (_allocFn or device.alloc)(bucket, mode)


def poolFree(buffer, nbytes, mode=device.SHARED):
    if not buffer:
        return
    bucket = bucketSize(nbytes)
    pool = _privatePool if mode == device.PRIVATE else _sharedPool
    pool.setdefault(bucket, []).append({"buffer": buffer, "bytes": bucket})


def poolStats():
    """src/pool.js:51-70"""
    sc = sum(len(b) for b in _sharedPool.values())
    pc = sum(len(b) for b in _privatePool.values())
    sb = sum(size * len(b) for size, b in _sharedPool.items())
    pb = sum(size * len(b) for size, b in _privatePool.items())
    return {
        "hits": _hits,
        "misses": _misses,
        "hitRate": _hits / ((_hits + _misses) or 1),
        "totalAllocated": _totalAllocated,
        "shared": {"count": sc, "bytes": sb},
        "private": {"count": pc, "bytes": pb},
    }


def poolFlush():
    stats = poolStats()
    _sharedPool.clear()
    _privatePool.clear()
    return stats


def poolDrain():
    global _hits, _misses, _totalAllocated
    result = poolFlush()
    _hits = _misses = _totalAllocated = 0
    return result
