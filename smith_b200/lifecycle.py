"""Tensor lifetime helpers -- the role of src/lifecycle.js in the reference.

dispose / retain reference counting, ``using`` scopes that release what was
allocated inside them, and the ``withNoAlloc`` guard.  Like the reference
(src/lifecycle.js:5-12) it knows nothing about the device: tensor.py plugs the
pool's free function in through ``setReleaseFn``.
"""
_releaseFn = lambda t: None
_scopeStack = []
_noAllocMode = False


def setReleaseFn(fn):
    global _releaseFn
    _releaseFn = fn


def dispose(t):
    """src/lifecycle.js:24-37"""
    if t is None or getattr(t, "_disposed", False):
        return
    rc = getattr(t, "_refCount", None)
    if rc is not None and rc > 1:
        t._refCount = rc - 1
        return
    t._disposed = True
    t._refCount = 0
    if t.buffer:
        _releaseFn(t)
        t.buffer = None
        t.data = None


def retain(t):
    """src/lifecycle.js:41-46"""
    if t is None:
        return t
    if getattr(t, "_refCount", None) is None:
        t._refCount = 1
    t._refCount += 1
    return t


def isDisposed(t):
    return bool(t is not None and getattr(t, "_disposed", False))


def using(fn):
    """Run fn; tensors created inside and not retained are released (src/lifecycle.js:65-77)."""
    scope = []
    _scopeStack.append(scope)
    try:
        return fn()
    finally:
        _scopeStack.pop()
        for t in scope:
            if not getattr(t, "_disposed", False):
                dispose(t)


def withNoAlloc(fn):
    """src/lifecycle.js:96-103"""
    global _noAllocMode
    _noAllocMode = True
    try:
        return fn()
    finally:
        _noAllocMode = False


def trackAllocation(t):
    """Called by tensor.create for every new tensor (src/lifecycle.js:107-118)."""
    if _noAllocMode:
        raise RuntimeError("Unexpected tensor allocation inside withNoAlloc()")
    if getattr(t, "_refCount", None) is None:
        t._refCount = 1
    t._disposed = False
    if _scopeStack:
        _scopeStack[-1].append(t)


def activeScopeDepth():
    return len(_scopeStack)
