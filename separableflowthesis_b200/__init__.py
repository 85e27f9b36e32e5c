"""B200 (sm_100a) implementation of SeparableFlow's memory-saving cost-volume separation.

``separableflowthesis_b200.MemorySaver`` exposes the five native ops under the names of the
reference's pybind11 module (libs/MemorySaver/src/MemorySaver_cuda.cpp:105-112);
``separableflowthesis_b200.functions`` holds the three autograd Functions of
libs/MemorySaver/functions/MemorySaver.py and ``separableflowthesis_b200.corr`` the call site
(core/corr.py:335-510).
"""
from . import ops as MemorySaver  # noqa: F401
from .functions import (  # noqa: F401
    ComputeMaxAvgFunction,
    ComputeMaxArgmaxAvgFunction,
    ComputeSelfCompressionFunction,
)
from .modules import ComputeMaxAvgModule  # noqa: F401
from .corr import AlternateCorrBlockSepflow, CorrBlock1D  # noqa: F401

__all__ = [
    "MemorySaver", "ComputeMaxAvgFunction", "ComputeMaxArgmaxAvgFunction",
    "ComputeSelfCompressionFunction", "ComputeMaxAvgModule", "AlternateCorrBlockSepflow", "CorrBlock1D",
]
