"""Collectives of the in-place family (reference: rtp/inplace/module/collectives.py): the same TP regions
and flat-buffer helpers, plus the blocking whole-buffer ring shifts."""
from ...module.collectives import *  # noqa: F401,F403
from ...module.collectives import (_CopyToModelParallelRegion, _GatherFromModelParallelRegion,  # noqa: F401
                                   _ReduceFromModelParallelRegion, _ShiftToModelParallelRegion, _gather, _reduce,
                                   _split)
from ...parallel.context import get_context
from ...parallel import ring as _ring


def _right_shift(input_, group=None):
    """Blocking hop r -> r+1 that replaces ``input_`` by the buffer of rank r-1 (chunked, no full temp)."""
    _ring.shift_inplace(get_context(group), input_, "up")
    return input_


def _left_shift(input_, group=None):
    """Blocking hop r -> r-1 that replaces ``input_`` by the buffer of rank r+1."""
    _ring.shift_inplace(get_context(group), input_, "down")
    return input_
