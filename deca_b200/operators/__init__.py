from .Op import Operator
from .GEMMTC import GEMMTC
from .FlashAttention import FlashAttention
from .Rowwise import RowwiseOperator, TOLERANCE
from .Softmax import Softmax
from .RMSNorm import RMSNorm

__all__ = ["Operator", "GEMMTC", "FlashAttention", "RowwiseOperator", "Softmax", "RMSNorm", "TOLERANCE"]
